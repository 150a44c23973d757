"""Tensor-parallel host logic on CPU: sharding of the packed layout and the all-reduce plumbing,
with world_size-2 gloo ranks.  The per-rank matmul is done by the CPU oracle (the checker), so
the test needs no GPU; on the GPU the same classes call the CUDA kernel."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bitween_b200 import QuantizedLinear, synth, tp
from helpers import from_bits, oracle_forward, to_np
from oracle import oracle


def _layer(seed, N, K, bits, g, bias):
    w = synth.normal(seed, (N, K), 0.02)
    q, s, z = oracle.quantize_rtn(w, oracle.F32, bits, g)
    ql = QuantizedLinear(K, N, bits, g, bias=bias)
    ql.qweight.copy_(torch.from_numpy(q))
    ql.scale.copy_(torch.from_numpy(s))
    ql.zero_point.copy_(torch.from_numpy(z))
    if bias:
        ql.bias.copy_(torch.from_numpy(synth.normal(seed + 1, (N,), 0.02)))
    return ql, w


def _oracle_matmul(x, qweight, scale, zero_point, bias, bits, group_size, **kw):
    x2 = x.reshape(-1, x.shape[-1])
    if kw.get("out_dtype") == torch.float32:
        # the library's fp32 output: the accumulator plus the bias, no 16-bit rounding
        _, acc = oracle_forward(x2, qweight, scale, zero_point, None, bits, group_size, want_acc=True)
        return acc if bias is None else acc + bias.float()
    return oracle_forward(x2, qweight, scale, zero_point, bias, bits, group_size)


def test_shards_equal_quantizing_the_sharded_weight():
    # groups never straddle a shard: shard(quantize(W)) == quantize(shard(W)) bit for bit
    for bits, g in ((4, 128), (8, 32), (2, 64)):
        ql, w = _layer(10 + bits, 64, 512, bits, g, True)
        for world in (2, 4):
            for rank in range(world):
                col = tp.shard_quantized_linear(ql, "column", rank, world)
                n = 64 // world
                q, s, z = oracle.quantize_rtn(w[rank * n:(rank + 1) * n], oracle.F32, bits, g)
                assert np.array_equal(col.qweight.numpy(), q)
                assert np.array_equal(to_np(col.scale), oracle.f16_bits(s))
                row = tp.shard_quantized_linear(ql, "row", rank, world)
                k = 512 // world
                q, s, z = oracle.quantize_rtn(np.ascontiguousarray(w[:, rank * k:(rank + 1) * k]), oracle.F32, bits, g)
                assert np.array_equal(row.qweight.numpy(), q)
                assert np.array_equal(to_np(row.zero_point), oracle.f16_bits(z.astype(np.float32)))
                assert (row.bias is not None) == (rank == 0)


def test_row_parallel_split_must_respect_groups_and_words():
    ql, _ = _layer(3, 8, 384, 4, 128, False)
    with pytest.raises(ValueError, match="group_size"):
        tp.shard_quantized_linear(ql, "row", 0, 2)          # 192 is not a multiple of 128
    with pytest.raises(ValueError):
        tp.shard_quantized_linear(ql, "column", 0, 3)       # 8 rows over 3 ranks
    with pytest.raises(ValueError):
        tp.shard_quantized_linear(ql, "diag", 0, 2)
    assert tp.check_row_parallel(28672, 4, 128, 8) == 3584  # Llama-3-70B down_proj over 8 GPUs
    f = tp.layer_shard_filter(1, 4)
    assert [i for i in range(10) if f(i, "x")] == [1, 5, 9]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tp._matmul = _oracle_matmul
        torch.manual_seed(0)
        up, _ = _layer(21, 96, 256, 4, 64, True)       # column-parallel
        down, _ = _layer(23, 64, 96, 8, 16, True)      # row-parallel (96/2 = 48 = 3 groups)
        x = torch.from_numpy(synth.normal(25, (5, 256), 1.0)).half()
        col = tp.ColumnParallelQuantizedLinear.from_full(up, rank, world)
        row = tp.RowParallelQuantizedLinear.from_full(down, rank, world)
        h = col(x)                                      # [5, 48] sharded
        assert tuple(h.shape) == (5, 96 // world)
        y = row(torch.relu(h))                          # all-reduce inside
        tp.check_same_across_ranks(y.shape)
        # fp32 partial sums on the wire, one fp16 rounding after the reduce
        row32 = tp.RowParallelQuantizedLinear.from_full(down, rank, world, reduce_dtype=torch.float32)
        y32 = row32(torch.relu(h))
        assert y32.dtype == torch.float16 and y32.shape == y.shape
        # single-process reference of the same two layers
        h_full = _oracle_matmul(x, up.qweight, up.scale, up.zero_point, up.bias, 4, 64)
        y_full = _oracle_matmul(torch.relu(h_full), down.qweight, down.scale, down.zero_point, down.bias, 8, 16)
        err = float((y.float() - y_full.float()).abs().max())
        rms = float(y_full.float().pow(2).mean().sqrt())
        gathered = tp.ColumnParallelQuantizedLinear.from_full(up, rank, world, gather_output=True)(x)
        ok_gather = bool(torch.equal(gathered, h_full))
        # a rank that disagrees on shapes is caught on the host, before any collective on data
        try:
            tp.check_same_across_ranks((5, 64 + rank))
            mismatch_caught = False
        except RuntimeError:
            mismatch_caught = True
        err32 = float((y32.float() - y_full.float()).abs().max())
        ret[rank] = (err, rms, ok_gather, mismatch_caught, err32)
    finally:
        dist.destroy_process_group()


def test_two_rank_column_then_row_parallel_matches_single_process():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, rms, ok_gather, mismatch_caught, err32 = ret[rank]
        # partial sums are rounded to fp16 before the all-reduce: 1e-2 * RMS(output) bar
        assert err <= 1e-2 * rms, (rank, err, rms)
        # with fp32 partials only the final rounding differs from the single-process result: one fp16 ulp
        assert err32 <= max(2.0 ** -10 * 4 * rms, 1e-3 * rms), (rank, err32, rms)
        assert ok_gather and mismatch_caught
