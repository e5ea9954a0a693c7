"""Child process of tests/test_gpu_multi.py: one rank of a column-parallel group.
Usage (under torch.distributed.run): multi_rank_worker.py {linear|decoder} OUT.json"""
import json
import os
import sys

import torch
import torch.distributed as dist


def _linear_case(ops, tp, comm, rank, world, gen, M):
    K, N, N2 = 1024, 256 * world, 128 * world
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda", generator=gen)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen)
    w2 = torch.randint(-127, 128, (N2, N), dtype=torch.int8, device="cuda", generator=gen)
    sw = torch.rand(N, device="cuda", generator=gen) * 9e-3 + 1e-3
    sw2 = torch.rand(N2, device="cuda", generator=gen) * 9e-3 + 1e-3
    sx = torch.rand(M, device="cuda", generator=gen) * 0.03 + 0.01
    # unsplit on this GPU
    y_full = ops.qgemm(a, w, x_scale=sx, w_scale=sw, out_dtype=torch.float16)
    s_full = ops.row_scale_local(y_full)
    q_full = ops.quantize_rows(y_full, s_full)
    z_full = ops.qgemm(q_full, w2, x_scale=s_full, w_scale=sw2, out_dtype=torch.float16)
    # split: shard -> gather fp16; local scales -> max over ranks -> int8 gather -> next shard reads slabs
    lin1 = tp.ColumnParallelQLinear(w, sw, None, comm)
    lin2 = tp.ColumnParallelQLinear(w2, sw2, None, comm)
    y_g = lin1.forward(a, sx)
    q_g, s_g = tp.quantize_rows_gathered(comm, y_g[rank])
    z_g = lin2.forward(q_g, s_g, a_gathered=True)
    torch.cuda.synchronize()
    acc = bool(torch.equal(tp.gathered_to_rowmajor(y_g), y_full))
    scale = bool(torch.equal(s_g, s_full)) and bool(torch.equal(tp.gathered_to_rowmajor(q_g), q_full))
    chain = bool(torch.equal(tp.gathered_to_rowmajor(z_g), z_full))
    return acc, scale, chain


def main():
    what, out_path = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("gloo")  # host channel only; the data path uses this library's communicator
    from bladedisc_b200 import ops, tp
    from bladedisc_b200.decoder import DecoderConfig, QuantDecoder
    comm = tp.Communicator.from_torch_distributed(torch.device("cuda", torch.cuda.current_device()))
    gen = torch.Generator(device="cuda").manual_seed(11)
    result = {}
    if what == "linear":
        result = {"acc_equal": True, "scale_equal": True, "chain_equal": True}
        for M, blocks in ((96, 1), (4608, 1), (4608, 2)):  # last: computed and gathered block of rows by block of rows
            tp.MAX_ROW_BLOCKS = blocks
            acc, scale, chain = _linear_case(ops, tp, comm, rank, world, gen, M)
            result["acc_equal"] &= acc
            result["scale_equal"] &= scale
            result["chain_equal"] &= chain
    else:
        cfg = DecoderConfig.tiny()
        cfg.heads = 8
        ids = torch.randint(0, cfg.vocab, (2, 20), device="cuda", generator=gen)
        one = QuantDecoder(cfg, None, seed=5)
        one.start(2, 32)
        ref_p = one.forward(ids[:, :19]).float()
        ref_d = one.forward(ids[:, 19:]).float()
        many = QuantDecoder(cfg, comm, seed=5)
        many.start(2, 32)
        got_p = many.forward(ids[:, :19]).float()
        got_d = many.forward(ids[:, 19:]).float()
        torch.cuda.synchronize()

        def close(x, y):  # attention runs per head group in a library kernel: allow its last-bit differences
            return float(((x - y).abs() <= 2e-3 + 2e-2 * y.abs()).float().mean().item())

        result["prefill_close"], result["decode_close"] = close(got_p, ref_p), close(got_d, ref_d)
    result["status"] = ops.kernel_status()
    flags = torch.tensor([1.0 if all(v is True or not isinstance(v, bool) for v in result.values()) else 0.0])
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        merged = dict(gathered[0])
        for r in gathered[1:]:
            for k, v in r.items():
                merged[k] = (merged[k] and v) if isinstance(v, bool) else (min(merged[k], v) if k.endswith("close") else max(merged[k], v))
        with open(out_path, "w") as f:
            json.dump(merged, f)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
