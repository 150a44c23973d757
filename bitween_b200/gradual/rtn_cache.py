"""Cache of RTN results for the gradual search.

The reference's precision search (bitween/gradual/precision_optimizer.py:146-166) tries, for
every block, each bit width against a sequence of group sizes, and its RTN wrapper
(bitween/gradual/base_wrapper.py:289-315) re-quantizes the block's unchanged weights from
scratch on every trial; nothing is kept.  Here the packed codes, scales and zero points of a
(weight, bits, group_size) triple are computed once and handed out again while the weight
tensor is unchanged.
"""
import collections
import threading

import torch


class RTNCache:
    """LRU cache `(weight storage, version, shape, dtype, device, bits, group_size) ->
    (qweight, scale, zero_point)`, bounded by the bytes it holds.

    A weight that is replaced, or modified in place through the parameter itself (optimizer
    steps, `with torch.no_grad(): w.add_(...)` -- anything that moves its version counter), gets
    a new key.  Edits made through `weight.data` bypass the version counter by design of torch
    and are NOT seen: call `clear()` after such edits.  Entries of freed weights age out.  The
    cached tensors are shared by every QuantizedLinear built from them: treat them as read-only.
    """

    def __init__(self, max_bytes=4 << 30):
        self.max_bytes = int(max_bytes)
        self._entries = collections.OrderedDict()
        self._bytes = 0
        self._lock = threading.Lock()
        self.hits = 0
        self.misses = 0

    @staticmethod
    def key(weight, bits, group_size):
        return (weight.data_ptr(), weight._version, tuple(weight.shape), weight.dtype, str(weight.device),
                int(bits), int(group_size))

    def get(self, weight, bits, group_size):
        k = self.key(weight, bits, group_size)
        with self._lock:
            hit = self._entries.get(k)
            if hit is None:
                self.misses += 1
                return None
            self._entries.move_to_end(k)
            self.hits += 1
            return hit

    def put(self, weight, bits, group_size, buffers):
        k = self.key(weight, bits, group_size)
        size = sum(t.numel() * t.element_size() for t in buffers)
        with self._lock:
            if k in self._entries:
                return
            self._entries[k] = tuple(buffers)
            self._bytes += size
            while self._bytes > self.max_bytes and len(self._entries) > 1:
                _, old = self._entries.popitem(last=False)
                self._bytes -= sum(t.numel() * t.element_size() for t in old)

    def clear(self):
        with self._lock:
            self._entries.clear()
            self._bytes = 0

    def __len__(self):
        return len(self._entries)

    @property
    def nbytes(self):
        return self._bytes


_default = RTNCache()


def default_cache():
    """The process-wide cache used by RTNWrapper unless it is given another one."""
    return _default
