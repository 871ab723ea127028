"""All-reduce of small bf16 tensors through peer memory (csrc/tpx_allreduce.cu) for the tensor-parallel decoder layers.

The reference has its own latency-oriented all-reduce between the ranks of one host (shared memory,
src/csrc/shm_coll.cpp, selected by USE_SHM_ALLREDUCE); this is its counterpart for GPUs of one NVLink domain. Each rank
owns an exchange buffer, a flag array and a small state block inside one symmetric-memory allocation (every rank can
address every rank's copy); torch.distributed only does the plumbing (allocation and address exchange). Tensors that do
not fit (more than MAX_ELEMS elements, not bf16, ...) go through the process group's own all-reduce."""
import ctypes
import os

import torch

from . import _lib

MAX_ELEMS = 1 << 20            # what the exchange buffer holds per call: 2 MiB of bf16
_BUF_ELEMS = 2 * MAX_ELEMS     # two halves, alternating by call
# Largest tensor sent through the peer kernel by default. Issued back to back between two GPUs the kernel beats NCCL at
# every size (8 KiB: 11 against 21 us, 1 MiB: 21 against 28 us), but inside a Llama-2-70B decode step at batch 64 (161 calls
# of 1 MiB between dependent kernels) the step was slower with it (25.6 against 24.9 ms; fewer CTAs made it worse), so
# tensors above this size stay with the library collective. TPX_ALLREDUCE_MAX_BYTES overrides.
AUTO_MAX_BYTES = int(os.environ.get("TPX_ALLREDUCE_MAX_BYTES", str(256 * 1024)))


class PeerAllReduce:
    def __init__(self, group):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        L = _lib.lib()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if not 2 <= self.world <= 8:
            raise _lib.TpxError("peer all-reduce serves 2 to 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device())
        flag_bytes = int(L.tpx_allreduce_flag_bytes())
        self._flag_off = _BUF_ELEMS * 2
        self._state_off = self._flag_off + flag_bytes
        self.mem = symm.empty(self._state_off + 256, dtype=torch.uint8, device=dev)
        self.mem.zero_()
        self.hdl = symm.rendezvous(self.mem, group)
        ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.buf_ptrs = (ctypes.c_uint64 * 8)(*(ptrs + [0] * (8 - len(ptrs))))
        self.flag_ptrs = (ctypes.c_uint64 * 8)(*([p + self._flag_off for p in ptrs] + [0] * (8 - len(ptrs))))
        self.state_ptr = ptrs[self.rank] + self._state_off
        torch.cuda.synchronize()
        dist.barrier(group)  # every rank's flags and state are zero before anyone signals

    def serves(self, t):
        return (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() % 8 == 0 and 0 < t.numel() <= MAX_ELEMS
                and t.numel() * 2 <= AUTO_MAX_BYTES and t.data_ptr() % 16 == 0)

    def __call__(self, t):
        _lib.check(_lib.lib().tpx_allreduce_bf16(t.data_ptr(), t.numel(), self.rank, self.world, self.buf_ptrs, self.flag_ptrs, self.state_ptr,
                                                 _BUF_ELEMS, _lib.stream()))
        return t

    def error_code(self):
        """Non-zero if a call gave up waiting for a peer (1 + the peer's rank); waits for the device."""
        torch.cuda.synchronize()
        return int(self.mem[self._state_off + 8:self._state_off + 12].view(torch.int32).item())


_instances = {}
_failed = set()


def get(group):
    """The peer all-reduce of `group`, or None when it is switched off (TPX_ALLREDUCE=nccl) or cannot be set up here."""
    if os.environ.get("TPX_ALLREDUCE", "peer") != "peer":
        return None
    key = id(group)
    if key in _failed:
        return None
    inst = _instances.get(key)
    if inst is None:
        try:
            inst = _instances[key] = PeerAllReduce(group)
        except Exception as e:  # no symmetric memory in this environment: the library collective serves
            import warnings
            warnings.warn(f"peer-memory all-reduce unavailable ({e!r}); using the process group's all-reduce")
            _failed.add(key)
            return None
    return inst


def release(group=None):
    """Drop the buffers (before the process group is destroyed)."""
    for k in list(_instances):
        if group is None or k == id(group):
            del _instances[k]
