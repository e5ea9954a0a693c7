"""Column-parallel configuration on one GPU: the gathered layouts, the two-pass
row quantization, the collective custom calls on a one-rank communicator, and
the decoder harness against a plain torch restatement.  (Two and more ranks:
tests/test_gpu_multi.py.)"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from bladedisc_b200 import ops as o
    return o


def _silu(x):
    return x / (1.0 + np.exp(-x))


@pytest.mark.parametrize("rows,cols,ld", [(5, 64, 64), (64, 1376, 2752), (300, 512, 1024), (33, 100, 203), (16, 4096, 8192)])
@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_two_pass_row_quantize(ops, rows, cols, ld, gated, dtype):
    rng = np.random.default_rng(rows + cols)
    buf = torch.from_numpy(rng.standard_normal((rows, ld)).astype(np.float32) * 3).to(dtype).cuda()
    gate = buf[:, :cols]
    up = buf[:, ld - cols:] if gated else None
    if gated and ld < 2 * cols:
        pytest.skip("halves overlap")
    g = gate.float().cpu().numpy().astype(np.float64)
    h = _silu(g) * up.float().cpu().numpy() if gated else g
    scale = ops.row_scale_local(gate, up)
    want_scale = np.maximum(np.abs(h).max(axis=1) / 127.0, np.finfo(np.float32).eps)
    assert np.allclose(scale.cpu().numpy(), want_scale, rtol=2e-6 if not gated else 1e-5)
    out = torch.full((rows + 2, cols + 16), 77, dtype=torch.int8, device="cuda")
    q = ops.quantize_rows(gate, scale, up, out=out[1:rows + 1, :cols])
    want = np.clip(np.rint(h / scale.cpu().numpy().astype(np.float64)[:, None]), -128, 127)
    diff = np.abs(q.cpu().numpy().astype(np.int32) - want.astype(np.int32))
    # with gating (approximate exp / reciprocal) a value may land one level off, but only a small share may
    # `want` divides in double: against it a float32 quotient on a rounding tie may land on the other level
    assert diff.max() <= 1 and (diff > 0).mean() < (1e-2 if gated else 1e-3), ((diff > 0).mean(), diff.max())
    assert np.abs(q.cpu().numpy()).max() == 127  # the row maximum lands on the last level
    q2, s2 = ops.quantize_rows_whole(gate, up)     # both passes in one kernel: the same bytes
    assert torch.equal(q2, q) and torch.equal(s2, scale)
    # the C oracle (which divides): the reciprocal form may land one level off on a small share of the values,
    # a few more with gating (approximate exp / reciprocal)
    from oracle import c
    oq, os_ = c.gated_quantize(gate.float().cpu().numpy(), up.float().cpu().numpy() if gated else None)
    odiff = np.abs(q.cpu().numpy().astype(np.int32) - oq.astype(np.int32))
    if gated:
        assert np.allclose(scale.cpu().numpy(), os_, rtol=1e-5) and odiff.max() <= 1 and (odiff > 0).mean() < 2e-3
    else:
        assert (scale.cpu().numpy() == os_).all() and odiff.max() <= 1 and (odiff > 0).mean() < 1e-3
    assert (out[0] == 77).all() and (out[rows + 1] == 77).all() and (out[:, cols:] == 77).all()


@pytest.mark.parametrize("rows,g,slab", [(7, 2, 128), (100, 4, 1024), (64, 8, 512), (300, 2, 2048)])
def test_norm_reads_gathered_slabs(ops, rows, g, slab):
    from bladedisc_b200 import tp
    cols = g * slab
    gen = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=gen, device="cuda").half()
    res = torch.randn(rows, cols, generator=gen, device="cuda").half()
    gamma = (1 + 0.1 * torch.randn(cols, generator=gen, device="cuda")).half()
    q0, s0, sum0 = ops.rmsnorm_dynamic_quant(x, gamma, 1e-5, residual=res)
    xg = tp.rowmajor_to_gathered(x, g)
    q1, s1, sum1 = ops.rmsnorm_dynamic_quant(xg, gamma, 1e-5, residual=res, x_gathered=True)
    assert torch.equal(q0, q1) and torch.equal(s0, s1) and torch.equal(sum0, sum1)
    assert torch.equal(tp.gathered_to_rowmajor(xg), x)
    from oracle import c
    assert (xg.cpu().numpy() == c.gathered_layout(x.cpu().numpy(), g)).all()
    y0 = ops.rmsnorm(x, gamma, 1e-5, residual=res)
    y1 = ops.rmsnorm(xg, gamma, 1e-5, residual=res, x_gathered=True)
    assert torch.equal(y0, y1)


def test_one_rank_communicator_and_collectives(ops):
    from bladedisc_b200 import tp, lib
    assert lib.load().disc_b200_nccl_available() > 0
    comm = tp.Communicator.single()
    buf = torch.arange(24, dtype=torch.float16, device="cuda").reshape(1, 4, 6).contiguous()
    want = buf.clone()
    comm.all_gather_(buf)
    t = torch.tensor([1.0, -2.0, 3.5], device="cuda")
    comm.all_reduce_max_(t)
    torch.cuda.synchronize()
    assert torch.equal(buf, want) and t.tolist() == [1.0, -2.0, 3.5]
    comm.close()


def test_ral_collective_calls_one_rank(ops):
    """ral_all_gather / ral_all_reduce / ral_async_collective_done and the fused
    disc_b200_qgemm_all_gather through the packed-argument dispatcher."""
    from bladedisc_b200 import ral, tp
    from bladedisc_b200.ral import MemRefSpec
    from oracle import c
    comm = tp.Communicator.single()
    side = torch.cuda.Stream()
    ctx = ral.RalContext(nccl_comm=comm.handle, comm_stream=side.cuda_stream)
    blob = ctx.attr_blob
    x = torch.randn(3, 8, device="cuda").half()
    groups = np.zeros((1, 1), dtype=np.int64)
    ag = blob({"all_gather_dim": 1, "replica_groups": groups, "is_async": True, "async_token_key": 5})
    y = ctx.call("ral_all_gather", "gpu", [("pvoid", 0), x, ("pvoid", ag)], [MemRefSpec("f16", 2)])
    z = ctx.call("ral_async_collective_done", "gpu",
                 [("pvoid", 0), y, ("pvoid", blob({"is_async": True, "async_token_key": 5}))], [MemRefSpec("f16", 2)])
    torch.cuda.synchronize()
    assert tuple(z.shape) == (3, 8) and torch.equal(z, x)
    r = ctx.call("ral_all_reduce", "gpu",
                 [("pvoid", 0), x.float(), ("pvoid", blob({"reduction_kind": "max", "is_async": False}))],
                 [MemRefSpec("f32", 2)])
    torch.cuda.synchronize()
    assert torch.equal(r, x.float())
    # a "done" without a collective in flight is an error, not a hang
    with pytest.raises(ral.RalError, match="token"):
        ctx.call("ral_async_collective_done", "gpu",
                 [("pvoid", 0), x, ("pvoid", blob({"is_async": True, "async_token_key": 9}))], [MemRefSpec("f16", 2)])
    # a replica group that does not match the communicator is refused
    with pytest.raises(ral.RalError, match="replica group"):
        bad = blob({"all_gather_dim": 0, "replica_groups": np.zeros((1, 2), dtype=np.int64), "is_async": False})
        ctx.call("ral_all_gather", "gpu", [("pvoid", 0), x, ("pvoid", bad)], [MemRefSpec("f16", 2)])
    # fused shard + gather
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (40, 256), dtype=np.int8)
    w = rng.integers(-127, 128, (96, 256), dtype=np.int8)
    sw = (rng.random(96) * 9e-3 + 1e-3).astype(np.float32)
    sx = (rng.random(40) * 0.03 + 0.01).astype(np.float32)
    bias = (rng.standard_normal(96) * 0.1).astype(np.float32)
    dev = lambda v: torch.from_numpy(v).cuda()
    f = lambda v: torch.tensor(float(v), dtype=torch.float32, device="cuda")
    sync = ("pvoid", blob({"activation": "none", "is_async": False}))
    args = [("pvoid", 0), dev(a), dev(w), dev(bias), dev(sx), dev(sw), f(0.05), sync]
    out = ctx.call("disc_b200_qgemm_all_gather", "gpu", args, [MemRefSpec("f16", 3)])
    acc = c.qgemm_acc(a, w)
    want, _ = c.qgemm_epilogue(acc, x_scale=sx, w_scale=sw, bias=bias)
    assert tuple(out.shape) == (1, 40, 96)
    assert np.allclose(out[0].float().cpu().numpy(), want, rtol=1e-2, atol=1e-3)
    # int8 result, gathered asynchronously, then fed to the next linear as a gathered activation
    later = ("pvoid", blob({"activation": "none", "is_async": True, "async_token_key": 1, "exact_division": True}))
    out8 = ctx.call("disc_b200_qgemm_all_gather", "gpu", args[:-1] + [later], [MemRefSpec("i8", 3)])
    out8 = ctx.call("ral_async_collective_done", "gpu",
                    [("pvoid", 0), out8, ("pvoid", blob({"is_async": True, "async_token_key": 1}))],
                    [MemRefSpec("i8", 3)])
    _, mid = c.qgemm_epilogue(acc, x_scale=sx, w_scale=sw, out_scale=np.float32(0.05), bias=bias, div_out=True)
    assert (out8[0].cpu().numpy() == mid).all()
    w2 = rng.integers(-127, 128, (48, 96), dtype=np.int8)
    sw2 = (rng.random(48) * 9e-3 + 1e-3).astype(np.float32)
    nxt = ctx.call("disc_b200_qgemm_all_gather", "gpu",
                   [("pvoid", 0), out8, dev(w2), ("m1df32", None), f(0.05), dev(sw2), f(1.0), sync],
                   [MemRefSpec("f16", 3)])
    want2, _ = c.qgemm_epilogue(c.qgemm_acc(mid, w2), x_scale=np.float32(0.05), w_scale=sw2)
    assert np.allclose(nxt[0].float().cpu().numpy(), want2, rtol=1e-2, atol=1e-3)
    ctx.close()
    comm.close()


def test_collective_call_without_communicator_is_an_error(ops):
    from bladedisc_b200 import ral
    from bladedisc_b200.ral import MemRefSpec
    ctx = ral.RalContext()
    x = torch.randn(3, 8, device="cuda").half()
    with pytest.raises(ral.RalError, match="communicator"):
        ctx.call("ral_all_gather", "gpu", [("pvoid", 0), x, ("pvoid", ctx.attr_blob({"all_gather_dim": 0}))],
                 [MemRefSpec("f16", 2)])
    ctx.close()


@pytest.mark.parametrize("layers", [1, 2])
def test_decoder_matches_torch_restatement(ops, layers):
    from bladedisc_b200.decoder import DecoderConfig, QuantDecoder, reference_forward
    cfg = DecoderConfig.tiny()
    cfg.layers = layers
    dec = QuantDecoder(cfg, None, seed=7)
    ids = torch.randint(0, cfg.vocab, (3, 24), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    dec.start(3, 32)
    got = dec.forward(ids).float()
    want = reference_forward(dec, ids).float()
    err = (got - want).abs()
    close = (err <= 1e-3 + 1e-2 * want.abs()).float().mean().item()
    if layers == 1:
        # the stated end-to-end bound (rtol 1e-2 / atol 1e-3) on all but the few values behind
        # an int8 rounding that fell the other way (exp in silu, fp16 rounding of a sum)
        assert close > 0.97, close
    else:
        # a flipped rounding in layer 1 perturbs every input of layer 2, whose roundings then
        # differ as any two runs of a quantized net differ: bound the error against the signal
        assert err.mean().item() < 0.01 * want.abs().mean().item()
    assert err.max().item() < 0.1
    assert ops.kernel_status() == 0


def test_decoder_decode_steps_extend_prefill(ops):
    """Prefill of S tokens followed by one decode step equals a prefill of S + 1
    tokens in the last position (same kernels, cache instead of recompute)."""
    from bladedisc_b200.decoder import DecoderConfig, QuantDecoder
    cfg = DecoderConfig.tiny()
    dec = QuantDecoder(cfg, None, seed=7)
    ids = torch.randint(0, cfg.vocab, (2, 17), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    dec.start(2, 32)
    full = dec.forward(ids).view(2, 17, -1)
    dec.start(2, 32)
    dec.forward(ids[:, :16])
    step = dec.forward(ids[:, 16:17]).view(2, 1, -1)
    err = (full[:, 16:17].float() - step.float()).abs()
    assert (err <= 2e-3 + 2e-2 * full[:, 16:17].float().abs()).float().mean() > 0.97


def test_row_blocks_and_strided_gathered_operand(ops):
    """Long inputs of a column-parallel linear are computed and gathered block of
    rows by block of rows; a block of rows of a gathered activation is a strided
    view that the linear reads in place."""
    from bladedisc_b200 import tp
    from oracle import c
    assert tp._row_blocks(16384, 4, max_blocks=4) == [(0, 4096), (4096, 8192), (8192, 12288), (12288, 16384)]
    assert tp._row_blocks(16384, 1, max_blocks=4) == [(0, 16384)] and tp._row_blocks(100, 8, max_blocks=4) == [(0, 100)]
    assert tp._row_blocks(16384, 4) == [(0, 16384)]  # off unless asked for
    blocks = tp._row_blocks(5000, 2, max_blocks=4)
    assert blocks[0][0] == 0 and blocks[-1][1] == 5000 and all(b[0] % 128 == 0 for b in blocks)
    rng = np.random.default_rng(9)
    g, M, slab, N = 2, 300, 256, 72
    a = rng.integers(-127, 128, (M, g * slab), dtype=np.int8)
    w = rng.integers(-127, 128, (N, g * slab), dtype=np.int8)
    gathered = torch.from_numpy(np.ascontiguousarray(a.reshape(M, g, slab).transpose(1, 0, 2))).cuda()
    want = c.qgemm_acc(a, w)
    for m0, m1 in ((0, 128), (128, 300), (37, 41)):
        got = ops.qgemm(gathered[:, m0:m1, :], torch.from_numpy(w).cuda(), out_dtype=torch.int32, a_gathered=True)
        assert (got.cpu().numpy() == want[m0:m1]).all()


@pytest.mark.parametrize("batch,seq,heads,dim,pos0", [(2, 5, 3, 64, 0), (1, 1, 4, 128, 17), (3, 40, 2, 32, 8)])
def test_rope_and_cache_append_match_the_elementwise_form(ops, batch, seq, heads, dim, pos0):
    from bladedisc_b200.decoder import DecoderConfig, QuantDecoder
    dec = QuantDecoder.__new__(QuantDecoder)  # only the table / rotation helpers are used
    dec.cfg = DecoderConfig(hidden=heads * dim, heads=heads)
    dec.device = torch.device("cuda")
    dec._cos = dec._sin = None
    cache_len = pos0 + seq + 3
    dec._rope_tables(cache_len)
    gen = torch.Generator(device="cuda").manual_seed(batch + seq)
    qkv = torch.randn(batch * seq, 3 * heads * dim, generator=gen, device="cuda").half()
    q, k, v = qkv.view(batch, seq, 3, heads, dim).unbind(dim=2)
    want_q, want_k = dec._rope(q, pos0), dec._rope(k, pos0)
    kc = torch.full((batch, heads, cache_len, dim), 7.0, dtype=torch.float16, device="cuda")
    vc = torch.full_like(kc, 7.0)
    work = qkv.clone()
    ops.rope_kv_append(work, kc, vc, dec._cos, dec._sin, batch, seq, pos0)
    got = work.view(batch, seq, 3, heads, dim)
    assert torch.equal(got[:, :, 0], want_q)
    assert torch.equal(got[:, :, 1], k) and torch.equal(got[:, :, 2], v)          # k, v of the input stay as they were
    # the C oracle (fp32 restatement, rounded to fp16 as the kernel stores it)
    from oracle import c
    pos = np.tile(np.arange(pos0, pos0 + seq), batch)
    oq = c.rope(q.float().cpu().numpy().reshape(batch * seq, heads, dim), pos, dec._cos.cpu().numpy(),
                dec._sin.cpu().numpy())
    assert (got[:, :, 0].float().cpu().numpy().reshape(batch * seq, heads, dim) == oq.astype(np.float16).astype(np.float32)).all()
    assert torch.equal(kc[:, :, pos0:pos0 + seq], want_k.transpose(1, 2))
    assert torch.equal(vc[:, :, pos0:pos0 + seq], v.transpose(1, 2))
    assert (kc[:, :, :pos0] == 7).all() and (kc[:, :, pos0 + seq:] == 7).all() and (vc[:, :, pos0 + seq:] == 7).all()
    dec._rope_tables(2 * cache_len)
    with pytest.raises(RuntimeError, match="fit the cache"):  # positions past the end of the cache are refused
        ops.rope_kv_append(work, kc, vc, dec._cos, dec._sin, batch, seq, cache_len)
