"""The quantized linear on host buffers (rows streamed in, multiplied, streamed out in chunks by the library's
own pipeline, disc_b200_host_linear_run) gives the bytes of the direct call on device buffers."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,chunk", [(1, 64), (300, 128), (1000, 256), (2048, 2048), (5000, 1024)])
@pytest.mark.parametrize("int8_out", [True, False])
def test_host_linear_equals_the_direct_call(M, chunk, int8_out):
    from bladedisc_b200 import ops
    from bladedisc_b200.host_api import HostQLinear
    from oracle import c
    K, N = 512, 384
    rng = np.random.default_rng(M + chunk)
    a = torch.from_numpy(rng.integers(-127, 128, (M, K), dtype=np.int8))
    w = torch.from_numpy(rng.integers(-127, 128, (N, K), dtype=np.int8)).cuda()
    sw = torch.from_numpy((rng.random(N) * 9e-3 + 1e-3).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32)).cuda()
    sx = torch.tensor([0.02], device="cuda")
    so = torch.tensor([0.05], device="cuda") if int8_out else None
    layer = HostQLinear(w, sw, sx, bias=bias, out_scale=so, chunk_rows=chunk, slots=3)
    a_pin = a.pin_memory()
    out = torch.full((M, N), 7, dtype=torch.int8 if int8_out else torch.float16).pin_memory()
    for _ in range(2):   # the staging buffers are reused
        layer(a_pin, out)
        torch.cuda.synchronize()
        want = ops.qgemm(a.cuda(), w, x_scale=sx, w_scale=sw, bias=bias, out_scale=so,
                         out_dtype=torch.int8 if int8_out else torch.float16)
        assert torch.equal(out, want.cpu())
    # inputs of four chunks and more begin and end with chunk / 4, chunk / 4, chunk / 2
    chunks = (M + chunk - 1) // chunk if M < 4 * chunk else 6 + (M - 2 * chunk + chunk - 1) // chunk
    assert layer.kernel_launches == 2 * chunks
    # and the direct call is the oracle's arithmetic (spot check of the first rows)
    acc = c.qgemm_acc(a[:8].numpy(), w.cpu().numpy())
    f_want, q_want = c.qgemm_epilogue(acc, x_scale=np.float32(0.02), w_scale=sw.cpu().numpy(),
                                      out_scale=np.float32(0.05) if int8_out else None, bias=bias.cpu().numpy(),
                                      div_out=int8_out)
    if int8_out:
        assert np.abs(out[:8].numpy().astype(int) - q_want.astype(int)).max() <= 1
    else:
        assert np.allclose(out[:8].float().numpy(), f_want, rtol=1e-2, atol=1e-3)
    layer.close()
    with pytest.raises(ValueError):
        layer(a_pin[:, :8], out)
