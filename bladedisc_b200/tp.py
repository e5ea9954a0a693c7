"""Column-parallel (N-split) linears over the GPUs of one box.

Rank ``r`` of ``g`` holds rows ``[r * N / g, (r + 1) * N / g)`` of a weight
``[N, K]`` with their scales and bias and computes ``Y_r = X W_r^T`` of shape
``[M, N / g]``; one all-gather makes ``[g, M, N / g]`` on every rank.  That is
the pattern of the reference's ``ral_all_gather`` custom call
(tao_compiler/mlir/ral/collective.cu.cc:226-309): NCCL concatenates rank-major,
so the gathered buffer is *not* the row-major ``[M, N]`` matrix.  Here it never
has to become one: the GEMM epilogue writes slot ``r`` of the gather buffer
directly, NCCL gathers in place, and the next linear (``ops.qgemm(...,
a_gathered=True)``) and the next norm (``x_gathered=True``) read the slabs where
they lie.

One process per GPU.  The communicator is made by this library's own NCCL
binding; the 128-byte id travels over whatever ``torch.distributed`` group the
processes already share (gloo is enough).
"""
import ctypes
from typing import List, Optional, Tuple

import torch

from . import lib as _lib


def column_share(n: int, world: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """Rows ``[begin, end)`` of an ``[N, K]`` weight that ``rank`` owns.

    Every rank gets the same count (the all-gather needs equal shares), a
    multiple of ``multiple`` (16: the TMA alignment of a slab of the gathered
    activation).  ``n`` must split that way."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    if n % (world * multiple) != 0:
        raise ValueError(f"{n} output channels do not split into {world} shares that are multiples of {multiple}")
    share = n // world
    return rank * share, (rank + 1) * share


def gathered_to_rowmajor(buf: torch.Tensor) -> torch.Tensor:
    """``[g, M, C]`` rank-major slabs -> the ``[M, g * C]`` matrix they stand for
    (a copy; the kernels never need it, tests and hosts at the end of a model do)."""
    g, m, c = buf.shape
    return buf.permute(1, 0, 2).reshape(m, g * c)


def rowmajor_to_gathered(x: torch.Tensor, world: int) -> torch.Tensor:
    """Inverse of :func:`gathered_to_rowmajor`."""
    m, n = x.shape
    if n % world:
        raise ValueError("columns do not split evenly")
    return x.reshape(m, world, n // world).permute(1, 0, 2).contiguous()


class Communicator:
    """An NCCL communicator of this library (``disc_b200_nccl_comm_create``)."""

    def __init__(self, rank: int, world: int, unique_id: bytes):
        if len(unique_id) != 128:
            raise ValueError("an NCCL unique id has 128 bytes")
        self.rank, self.world = rank, world
        self._lib = _lib.load()
        handle = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(unique_id, 128)
        _lib.check(self._lib.disc_b200_nccl_comm_create(buf, world, rank, ctypes.byref(handle)))
        self.handle = handle.value

    @staticmethod
    def new_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        _lib.check(_lib.load().disc_b200_nccl_unique_id(buf))
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, device: torch.device, group=None) -> "Communicator":
        """Rank 0 makes the id; it reaches the others through ``torch.distributed``."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        torch.cuda.set_device(device)
        box: List[Optional[bytes]] = [cls.new_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(rank, world, box[0])

    @classmethod
    def single(cls) -> "Communicator":
        """A one-rank communicator (the same code path on one GPU)."""
        return cls(0, 1, cls.new_unique_id())

    def all_gather_(self, buf: torch.Tensor) -> torch.Tensor:
        """In place: ``buf`` is ``[world, ...]`` and slot ``rank`` holds this rank's share."""
        if buf.shape[0] != self.world or not buf.is_contiguous():
            raise ValueError("gather buffer must be contiguous [world, ...]")
        share = buf[self.rank]
        nbytes = share.numel() * share.element_size()
        stream = torch.cuda.current_stream(buf.device).cuda_stream
        _lib.check(self._lib.disc_b200_all_gather(self.handle, share.data_ptr(), buf.data_ptr(), nbytes, stream))
        return buf

    def all_gather_rows_(self, buf: torch.Tensor, row0: int, rows: int) -> torch.Tensor:
        """In place, rows ``[row0, row0 + rows)`` of every slot of ``buf [world, M, C]`` only."""
        if buf.dim() != 3 or buf.shape[0] != self.world or not buf.is_contiguous():
            raise ValueError("gather buffer must be contiguous [world, M, C]")
        row_bytes = buf.shape[2] * buf.element_size()
        stream = torch.cuda.current_stream(buf.device).cuda_stream
        _lib.check(self._lib.disc_b200_all_gather_rows(self.handle, buf.data_ptr(), self.world,
                                                       buf.shape[1] * row_bytes, row0 * row_bytes, rows * row_bytes,
                                                       stream))
        return buf

    def all_reduce_max_(self, t: torch.Tensor) -> torch.Tensor:
        """In place elementwise maximum over the ranks (float32)."""
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError("all_reduce_max_ takes a contiguous float32 tensor")
        stream = torch.cuda.current_stream(t.device).cuda_stream
        _lib.check(self._lib.disc_b200_all_reduce_f32(self.handle, t.data_ptr(), t.data_ptr(), t.numel(), 2, stream))
        return t

    def close(self) -> None:
        if self.handle:
            self._lib.disc_b200_nccl_comm_destroy(self.handle)
            self.handle = None


class ColumnParallelQLinear:
    """One rank's shard of a W8A8 linear with per-channel weight scales.

    ``forward`` takes the int8 activation (row-major ``[M, K]`` or gathered
    ``[g, M, K / g]``) with its per-row scales and returns the gathered fp16
    output ``[g, M, N / g]`` (``gather=True``) or just the local ``[M, N / g]``
    (``gather=False``: the consumer works on the local columns, e.g. attention
    heads or the SwiGLU product)."""

    def __init__(self, wq: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor],
                 comm: Optional[Communicator], rows: Optional[Tuple[int, int]] = None):
        world = comm.world if comm else 1
        rank = comm.rank if comm else 0
        if rows is None:
            rows = column_share(wq.shape[0], world, rank)
        b, e = rows
        self.comm = comm
        self.world, self.rank = world, rank
        self.wq = wq[b:e].contiguous()
        self.w_scale = w_scale[b:e].contiguous()
        self.bias = bias[b:e].contiguous() if bias is not None else None
        self.n_local = e - b
        # set once the weights are final and the stream that made them has been synchronised:
        # the few-row kernels then fetch them while the kernel before them still runs
        self.weights_static = False

    def forward(self, xq: torch.Tensor, x_scale: torch.Tensor, *, a_gathered: bool = False, gather: bool = True,
                act: Optional[str] = None) -> torch.Tensor:
        from . import ops
        m = xq.shape[1] if a_gathered else xq.shape[0]
        if not gather:
            return ops.qgemm(xq, self.wq, x_scale=x_scale, w_scale=self.w_scale, bias=self.bias, act=act,
                             out_dtype=torch.float16, a_gathered=a_gathered, weights_static=self.weights_static)
        buf = torch.empty((self.world, m, self.n_local), dtype=torch.float16, device=xq.device)
        blocks = _row_blocks(m, self.world)
        if len(blocks) == 1:
            ops.qgemm(xq, self.wq, x_scale=x_scale, w_scale=self.w_scale, bias=self.bias, act=act,
                      out_dtype=torch.float16, out=buf[self.rank], a_gathered=a_gathered,
                      weights_static=self.weights_static)
            if self.world > 1:
                self.comm.all_gather_(buf)
            return buf
        # Long inputs go block of rows by block of rows: while NCCL gathers one block on the
        # communication stream the kernel computes the next one.
        pipe = _Overlap(xq.device)
        for m0, m1 in blocks:
            a_blk = xq[:, m0:m1, :] if a_gathered else xq[m0:m1]
            s_blk = x_scale[m0:m1] if x_scale.numel() == m else x_scale
            ops.qgemm(a_blk, self.wq, x_scale=s_blk, w_scale=self.w_scale, bias=self.bias, act=act,
                      out_dtype=torch.float16, out=buf[self.rank, m0:m1], a_gathered=a_gathered,
                      weights_static=self.weights_static)
            pipe.after_compute(lambda m0=m0, m1=m1: self.comm.all_gather_rows_(buf, m0, m1 - m0))
        pipe.join()
        return buf


# Most row blocks a long input is cut into so that the gather of one block overlaps the
# computation of the next (1 = compute everything, then gather).  Measured on 4 B200s with
# the 7B-shaped prefill (8 x 2048 tokens, 8 layers): 21.7 ms with 1 block, 26.1 ms with 2,
# 30.2 ms with 4 -- the grouped broadcasts a row range needs are slower than one all-gather,
# the smaller GEMMs less efficient, and NCCL's kernels take SMs from them -- so the default
# is off.
MAX_ROW_BLOCKS = 1


def _row_blocks(m: int, world: int, min_rows: int = 2048, max_blocks: Optional[int] = None):
    """Row ranges for overlapping gathers with compute: one block unless there are ranks to talk
    to and enough rows for every block to stay an efficient GEMM."""
    if max_blocks is None:
        max_blocks = MAX_ROW_BLOCKS
    n = 1 if world <= 1 else max(1, min(max_blocks, m // min_rows))
    step = -(-m // n)
    step = -(-step // 128) * 128  # whole output tiles
    return [(b, min(b + step, m)) for b in range(0, m, step)]


class _Overlap:
    """Runs communication on a side stream behind the compute stream's progress."""
    _streams = {}

    def __init__(self, device):
        self.main = torch.cuda.current_stream(device)
        key = (device.index, self.main.cuda_stream)
        if key not in _Overlap._streams:
            _Overlap._streams[key] = torch.cuda.Stream(device)
        self.side = _Overlap._streams[key]
        self.side.wait_stream(self.main)  # the buffers exist before the side stream touches them

    def after_compute(self, fn):
        ev = torch.cuda.Event()
        ev.record(self.main)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            fn()

    def join(self):
        self.main.wait_stream(self.side)


def quantize_rows_gathered(comm: Optional[Communicator], gate: torch.Tensor, up: Optional[torch.Tensor] = None):
    """Per-row dynamic int8 quantization of ``h = silu(gate) * up`` (``h = gate``
    without ``up``) whose columns are spread over the ranks: local row maxima,
    maximum over the ranks, quantize into this rank's slot, all-gather.
    Returns ``(q [g, M, C] int8, row_scale [M])``."""
    from . import ops
    world = comm.world if comm else 1
    rank = comm.rank if comm else 0
    m, c = gate.shape
    if world == 1:  # the rows are whole here: scale and quantize in one kernel
        buf = torch.empty((1, m, c), dtype=torch.int8, device=gate.device)
        _, scale = ops.quantize_rows_whole(gate, up, out=buf[0])
        return buf, scale
    scale = ops.row_scale_local(gate, up)
    if world > 1:
        comm.all_reduce_max_(scale)
    buf = torch.empty((world, m, c), dtype=torch.int8, device=gate.device)
    blocks = _row_blocks(m, world)
    if len(blocks) == 1:
        ops.quantize_rows(gate, scale, up, out=buf[rank])
        if world > 1:
            comm.all_gather_(buf)
        return buf, scale
    pipe = _Overlap(gate.device)
    for m0, m1 in blocks:
        ops.quantize_rows(gate[m0:m1], scale[m0:m1], None if up is None else up[m0:m1], out=buf[rank, m0:m1])
        pipe.after_compute(lambda m0=m0, m1=m1: comm.all_gather_rows_(buf, m0, m1 - m0))
    pipe.join()
    return buf, scale
