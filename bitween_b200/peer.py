"""All-reduce of row-parallel partial outputs over peer memory (one node, one process per GPU),
the NCCL-free collective behind `RowParallelQuantizedLinear(collective="peer")`.

The reference is single-GPU; this belongs to the tensor-parallel layer of this library.  Every
rank's quantized matmul writes its partial sums straight into a buffer the other GPUs have mapped
through CUDA IPC, and one kernel per rank (C ABI: bw_peer_allreduce_f16) waits for all partials,
adds them in rank order and writes the fp16 sums locally -- one flag round trip and one pass of
peer loads instead of a library collective, which is what a decode step's 1 MiB all-reduce,
bound by latency, is short of.  Plain peer loads and stores; no multicast object is created.
"""
import ctypes

import torch
import torch.distributed as dist

from .kernels import _lib


class _RawCudaBuffer:
    """A device allocation that is not torch's, exposed through __cuda_array_interface__."""

    def __init__(self, ptr, nbytes):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerAllReduce:
    """Two partial-sum buffers of `max_elems` fp16 values per rank plus the flag array, mapped on
    every rank of `group` (all on one node).  Construction is collective (handles are exchanged
    with all_gather_object).  `partial(M, N)` returns this rank's buffer for the next call as an
    fp16 [M, N] tensor for the matmul to write into; `allreduce(out)` then sums it over the ranks
    into `out`.  Calls must be issued in the same order on every rank, on one stream per rank."""

    def __init__(self, max_elems, group=None, device=None, algo="auto"):
        if not dist.is_initialized():
            raise RuntimeError("PeerAllReduce needs an initialised process group")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerAllReduce serves at most 8 ranks (one node)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_elems = (int(max_elems) + 7) // 8 * 8
        if algo not in ("auto", "one_shot", "two_shot"):
            raise ValueError("algo must be 'auto', 'one_shot' or 'two_shot'")
        # one-shot: every rank reads every partial (world-1 times the data per rank, one barrier);
        # two-shot: reduce one slice each, publish, collect (2*(world-1)/world of the data, two barriers).
        # At the 1 MiB of a decode step the second barrier costs more than the bytes it saves (8 GPUs:
        # 21 us one-shot, 32 us two-shot, 34 us NCCL), so "auto" is one-shot up to 4 MiB and two-shot beyond.
        self.algo = algo
        self.two_shot = algo == "two_shot"
        L = _lib.lib()
        self._L = L
        self._local, self._opened = [], []
        nbytes = self.max_elems * 2
        with torch.cuda.device(self.device):
            # Every step that can fail locally is followed by an agreement over the group, so that a
            # failure on one rank raises on all of them instead of leaving the others in a collective.
            mine, err = [], None
            try:
                slice_bytes = ((self.max_elems // 8 + self.world - 1) // self.world) * 16
                mine = [self._alloc(nbytes), self._alloc(nbytes), self._alloc(L.bw_peer_flag_bytes()),
                        self._alloc(slice_bytes), self._alloc(slice_bytes)]
            except Exception as e:   # noqa: BLE001
                err = e
            self._agree(err, "allocating the peer buffers")
            gathered = [None] * self.world
            dist.all_gather_object(gathered, [h for (_, h) in mine], group=group)
            # ptrs[i][r]: this process's mapping of rank r's allocation i (0, 1: partial buffers, 2: flags,
            # 3, 4: reduced slices of the two-shot form)
            self._ptrs = [[None] * self.world for _ in range(5)]
            try:
                for r in range(self.world):
                    for i in range(5):
                        if r == self.rank:
                            self._ptrs[i][r] = mine[i][0]
                        else:
                            p = ctypes.c_void_p()
                            _lib.check(L.bw_peer_open(gathered[r][i], ctypes.byref(p)))
                            self._opened.append(p.value)
                            self._ptrs[i][r] = p.value
            except Exception as e:   # noqa: BLE001
                err = e
            self._agree(err, "mapping the peers' buffers (CUDA IPC)")
            self._state = torch.zeros(L.bw_peer_state_bytes(), dtype=torch.uint8, device=self.device)
        self._views = [torch.as_tensor(_RawCudaBuffer(mine[i][0], nbytes), device=self.device).view(torch.float16) for i in (0, 1)]
        self._arrays = [(ctypes.c_void_p * self.world)(*self._ptrs[i]) for i in range(5)]
        self._next = 0
        self._pending = None
        dist.barrier(group=group)          # every rank has mapped everything before the first call

    def _agree(self, err, what):
        ok = torch.tensor([0 if err is not None else 1], device=self.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            for p in self._opened:
                self._L.bw_peer_close(p)
            for p in self._local:
                self._L.bw_peer_free(p)
            self._opened, self._local = [], []
            raise RuntimeError(f"PeerAllReduce: {what} failed on " + ("this rank: " + repr(err) if err is not None else "another rank"))

    def _alloc(self, nbytes):
        p = ctypes.c_void_p()
        h = ctypes.create_string_buffer(64)
        _lib.check(self._L.bw_peer_alloc(nbytes, ctypes.byref(p), h))
        self._local.append(p.value)
        return p.value, h.raw

    def partial(self, M, N):
        """This rank's partial-sum buffer for the next all-reduce, as a contiguous fp16 [M, N] view."""
        if M * N > self.max_elems or (M * N) % 8 != 0:
            raise ValueError(f"{M}x{N} values do not fit the peer buffers ({self.max_elems}) or are not a multiple of 8")
        self._pending = (self._next, M * N)
        return self._views[self._next][:M * N].view(M, N)

    def allreduce(self, out):
        """Sums the buffer handed out by the last `partial` call over the ranks into `out` (fp16, contiguous)."""
        if self._pending is None:
            raise RuntimeError("call partial() and fill the buffer first")
        which, count = self._pending
        if out.dtype != torch.float16 or not out.is_contiguous() or out.numel() != count or out.device != self.device:
            raise ValueError("`out` must be a contiguous fp16 tensor of the partial's size on this rank's device")
        with torch.cuda.device(self.device):
            if self.two_shot or (self.algo == "auto" and count * 2 > (4 << 20) and self.world > 2):
                rc = self._L.bw_peer_allreduce2_f16(self._arrays[which], self._arrays[3 + which], self._arrays[2], self.rank,
                                                    self.world, _lib.ptr(out), count, _lib.ptr(self._state),
                                                    _lib.stream_ptr(self.device))
            else:
                rc = self._L.bw_peer_allreduce_f16(self._arrays[which], self._arrays[2], self.rank, self.world, _lib.ptr(out),
                                                   count, _lib.ptr(self._state), _lib.stream_ptr(self.device))
        _lib.check(rc)
        self._pending = None
        self._next ^= 1
        return out

    def close(self):
        """Collective: unmaps the peers' buffers and frees this rank's (after all ranks are done with them)."""
        if self._L is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self._L.bw_peer_close(p)
            dist.barrier(group=self.group)
            self._views = []
            for p in self._local:
                self._L.bw_peer_free(p)
        self._opened, self._local, self._L = [], [], None
