"""Tensor-parallel sharding of QuantizedLinear layers over the GPUs of one node, and
layer-wise sharding of RTN quantization.

The reference has no distributed code at all; this module adds the Megatron-style split that
the packed layout allows without re-quantizing:

  column-parallel (q/k/v, gate/up): split out_features -> contiguous ROW blocks of
      qweight [N/tp, K*bits/32], scale / zero_point [N/tp, K/g], bias [N/tp]; the input is
      replicated and the output stays sharded (it feeds the next row-parallel layer).
  row-parallel (o_proj, down_proj): split in_features -> COLUMN blocks qweight[:, (K/tp)*bits/32],
      scale / zero_point[:, (K/tp)/g]; needs (K/tp) % group_size == 0 and (K/tp) % (32/bits) == 0
      so that no group and no packed word straddles two ranks; each rank produces a partial
      [M, N] that one all-reduce (NCCL over NVLink / NVSwitch) sums.  The bias is added on
      rank 0 only, i.e. exactly once.

Groups never straddle a shard, so quantize-then-shard equals shard-then-quantize bit for bit.
One process per GPU; `torch.distributed` (backend "nccl") is the plumbing.
"""
import torch
import torch.distributed as dist
import torch.nn as nn

from .kernels.cuda_loader import quantized_matmul_cuda
from .modules import QuantizedLinear


def _matmul(*args, **kwargs):
    """Indirection point: the GPU kernel call (tests on CPU ranks substitute a checker here)."""
    return quantized_matmul_cuda(*args, **kwargs)


def check_row_parallel(in_features, bits, group_size, world):
    """Raises ValueError unless in_features splits over `world` ranks on group and word boundaries."""
    if in_features % world != 0:
        raise ValueError(f"in_features={in_features} is not divisible by tensor-parallel size {world}")
    k = in_features // world
    if k % group_size != 0:
        raise ValueError(f"row-parallel shard of {k} input features is not a multiple of group_size={group_size}")
    if k % (32 // bits) != 0:
        raise ValueError(f"row-parallel shard of {k} input features is not a multiple of {32 // bits} codes per word")
    return k


def shard_quantized_linear(layer: QuantizedLinear, mode: str, rank: int, world: int) -> QuantizedLinear:
    """Returns the rank's shard of `layer` as a new QuantizedLinear (buffers are copies)."""
    if mode not in ("column", "row"):
        raise ValueError("mode must be 'column' or 'row'")
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    N, K, bits, g = layer.out_features, layer.in_features, layer.bits, layer.group_size
    vpi = 32 // bits
    if mode == "column":
        if N % world != 0:
            raise ValueError(f"out_features={N} is not divisible by tensor-parallel size {world}")
        n = N // world
        out = QuantizedLinear(K, n, bits, g, bias=layer.bias is not None)
        rows = slice(rank * n, (rank + 1) * n)
        out.qweight = layer.qweight[rows].contiguous()
        out.scale = layer.scale[rows].contiguous()
        out.zero_point = layer.zero_point[rows].contiguous()
        if layer.bias is not None:
            out.bias = layer.bias[rows].contiguous()
        return out
    k = check_row_parallel(K, bits, g, world)
    out = QuantizedLinear(k, N, bits, g, bias=layer.bias is not None and rank == 0)
    out.qweight = layer.qweight[:, rank * (k // vpi):(rank + 1) * (k // vpi)].contiguous()
    out.scale = layer.scale[:, rank * (k // g):(rank + 1) * (k // g)].contiguous()
    out.zero_point = layer.zero_point[:, rank * (k // g):(rank + 1) * (k // g)].contiguous()
    if layer.bias is not None and rank == 0:
        out.bias = layer.bias.clone()
    return out


class ColumnParallelQuantizedLinear(nn.Module):
    """Holds rows [rank*N/tp, (rank+1)*N/tp) of a QuantizedLinear; no communication.
    `gather_output=True` all-gathers the sharded outputs along the last dimension."""

    def __init__(self, shard: QuantizedLinear, group=None, gather_output=False):
        super().__init__()
        self.shard = shard
        self.group = group
        self.gather_output = gather_output

    @classmethod
    def from_full(cls, layer, rank, world, group=None, gather_output=False):
        return cls(shard_quantized_linear(layer, "column", rank, world), group, gather_output)

    def forward(self, x):
        s = self.shard
        y = _matmul(x, s.qweight, s.scale, s.zero_point, s.bias, s.bits, s.group_size)
        if self.gather_output and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            parts = [torch.empty_like(y) for _ in range(dist.get_world_size(self.group))]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelQuantizedLinear(nn.Module):
    """Holds input columns [rank*K/tp, (rank+1)*K/tp) of a QuantizedLinear; the input is the
    matching slice of the activations and the partial outputs are summed with one all-reduce.

    `overlap_chunks` > 1 splits the tokens into that many chunks and runs the all-reduce of chunk
    i on a second stream while the GEMM of chunk i+1 runs (worth it for prefill, where the
    all-reduce moves tens of MB; a decode step's 1 MiB all-reduce is bound by latency, not
    bandwidth, and stays one piece).  `reduce_dtype=torch.float32` makes every rank emit its
    partial sums unrounded and rounds once after the reduce -- the reference's single fp16
    rounding -- at twice the bytes on the wire; the default sums fp16 partials (one extra
    rounding per rank, within the 1e-2 * RMS bar at 8 ranks).  `peer` (a `PeerAllReduce`) replaces
    the NCCL all-reduce of outputs that fit its buffers by the peer-memory kernel."""

    def __init__(self, shard: QuantizedLinear, group=None, overlap_chunks=1, reduce_dtype=None, peer=None):
        super().__init__()
        self.shard = shard
        self.group = group
        self.overlap_chunks = int(overlap_chunks)
        self.reduce_dtype = reduce_dtype
        self.peer = peer          # a bitween_b200.peer.PeerAllReduce shared by the layers of a model, or None (NCCL)
        self._comm_stream = None

    @classmethod
    def from_full(cls, layer, rank, world, group=None, overlap_chunks=1, reduce_dtype=None, peer=None):
        return cls(shard_quantized_linear(layer, "row", rank, world), group, overlap_chunks, reduce_dtype, peer)

    def _partial(self, x, out=None):
        s = self.shard
        kw = {} if self.reduce_dtype is None else {"out_dtype": self.reduce_dtype}
        if out is not None:
            kw["out"] = out
        return _matmul(x, s.qweight, s.scale, s.zero_point, s.bias, s.bits, s.group_size, **kw)

    def forward(self, x_shard):
        s = self.shard
        if x_shard.shape[-1] != s.in_features:
            raise ValueError(f"row-parallel input has {x_shard.shape[-1]} features, this rank holds {s.in_features}")
        distributed = dist.is_initialized() and dist.get_world_size(self.group) > 1
        x2 = x_shard.reshape(-1, s.in_features)
        M = x2.shape[0]
        chunks = min(self.overlap_chunks, M) if distributed and x2.is_cuda else 1
        if (distributed and self.peer is not None and self.reduce_dtype is None and x2.is_cuda
                and (M * s.out_features) % 8 == 0 and M * s.out_features <= self.peer.max_elems):
            # the matmul writes its partial sums into peer-mapped memory and one kernel sums them over
            # the ranks: no library collective (a decode step's all-reduce is bound by latency)
            self._partial(x2, out=self.peer.partial(M, s.out_features))
            y = torch.empty((M, s.out_features), dtype=torch.float16, device=x2.device)
            self.peer.allreduce(y)
            y = y.reshape(*x_shard.shape[:-1], s.out_features)
        elif chunks <= 1:
            y = self._partial(x_shard)
            if distributed:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        else:
            # GEMM of chunk i+1 (this stream) while chunk i is being reduced (second stream)
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=x2.device)
            dt = self.reduce_dtype or torch.float16
            y = torch.empty((M, s.out_features), dtype=dt, device=x2.device)
            main = torch.cuda.current_stream(x2.device)
            bounds = [M * i // chunks for i in range(chunks + 1)]
            for i in range(chunks):
                lo, hi = bounds[i], bounds[i + 1]
                self._partial(x2[lo:hi], out=y[lo:hi])
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(done)
                    dist.all_reduce(y[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
            main.wait_stream(self._comm_stream)
            y.record_stream(self._comm_stream)
            y = y.reshape(*x_shard.shape[:-1], s.out_features)
        if self.reduce_dtype is not None and self.reduce_dtype != torch.float16:
            y = y.to(torch.float16)
        return y


def layer_shard_filter(rank: int, world: int):
    """`layer_filter` for Bitween.quantize: rank r quantizes layers r, r+world, ... (layers are
    independent, so RTN quantization shards over GPUs with no communication)."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    return lambda index, name: index % world == rank


def check_same_across_ranks(values, group=None):
    """Host-side consistency check before a collective: every rank must agree on `values`
    (a tuple of ints, e.g. shapes).  Raises RuntimeError on the ranks that differ from rank 0."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    mine = [int(v) for v in values]
    gathered = [None] * dist.get_world_size(group)
    dist.all_gather_object(gathered, mine, group=group)
    if any(g != gathered[0] for g in gathered):
        raise RuntimeError(f"tensor-parallel ranks disagree: {gathered}")
