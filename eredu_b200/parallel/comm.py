"""Symmetric peer memory for one parallel group: allocation, CUDA-IPC exchange, tensor views.

One process per GPU. The buffer is a raw ``cudaMalloc`` allocation (so that its IPC handle maps the whole
region), zeroed, exchanged with ``torch.distributed.all_gather_object`` and mapped into every peer. Tensor views
of regions are created through ``__cuda_array_interface__`` (no copy).
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p, POINTER

import torch

from ..ops import native
from ..ops.native import I, L, P

native.register("eredu_peer_alloc", I, [L, POINTER(c_void_p)])
native.register("eredu_peer_free", I, [P])
native.register("eredu_ipc_handle_bytes", I, [])
native.register("eredu_ipc_get_handle", I, [P, P])
native.register("eredu_ipc_open", I, [P, POINTER(c_void_p)])
native.register("eredu_ipc_close", I, [P])
native.register("eredu_comm_create", P, [POINTER(c_void_p), I, I, L, L, P])
native.register("eredu_comm_destroy", None, [P])
native.register("eredu_comm_buffer_bytes", L, [L, L])
native.register("eredu_comm_init_buffer", I, [P, L, L])
native.register("eredu_comm_out_offset", L, [P])
native.register("eredu_comm_data_offset", L, [P, I, I])
native.register("eredu_allreduce_twoshot", I, [P, L, P, P, P, I, I, I, I, P, P])
native.register("eredu_allreduce_ll", I, [P, P, I, P, I, P, P, I, I, I, P, P])
native.register("eredu_allgather", I, [P, P, L, I, P, P])
native.register("eredu_peer_barrier", I, [P, P, P])
native.register("eredu_gemm_bf16_comm", I, [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, I, I, P, P, I,
                                             ctypes.c_float, I, P, P])


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device pointer."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int16: "<i2", torch.float16: "<f2"}


def view_raw(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """Tensor aliasing raw device memory (bf16 goes through an int16 view)."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_RawCuda(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    return torch.as_tensor(_RawCuda(ptr, shape, _TYPESTR[dtype]), device=device)


class PeerGroup:
    """Symmetric buffer of one group + the host ``PeerComm`` handed to the fused kernels."""

    def __init__(self, group, device: torch.device, slot_bytes: int, out_bytes: int, x_bytes: int = 0):
        import torch.distributed as dist

        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        lib = native.lib()
        self.lib = lib
        out_total = ((out_bytes + 255) // 256 * 256) + ((x_bytes + 255) // 256 * 256)
        self.bytes = int(lib.eredu_comm_buffer_bytes(slot_bytes, out_total))
        # Guard words in front of and behind the symmetric buffer: peers write into this allocation with plain stores, so
        # an index error of a remote kernel would otherwise corrupt silently. `check_canaries` (called on close and by
        # tests) finds a store that left the buffer.
        alloc = c_void_p()
        native.check(lib.eredu_peer_alloc(self.bytes + 2 * self.GUARD, ctypes.byref(alloc)), "eredu_peer_alloc")
        self._alloc = alloc.value
        self.own = self._alloc + self.GUARD
        for off in (0, self.GUARD + self.bytes):
            view_raw(self._alloc + off, (self.GUARD // 4,), torch.int32, device).fill_(self.CANARY)
        native.check(lib.eredu_comm_init_buffer(self.own, slot_bytes, out_total), "eredu_comm_init_buffer")
        hbytes = lib.eredu_ipc_handle_bytes()
        handle = ctypes.create_string_buffer(hbytes)
        native.check(lib.eredu_ipc_get_handle(self._alloc, handle), "cudaIpcGetMemHandle")
        handles = [None] * self.size
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.bases = []
        self._opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.own)
                continue
            p = c_void_p()
            native.check(lib.eredu_ipc_open(ctypes.create_string_buffer(h, hbytes), ctypes.byref(p)),
                         f"cudaIpcOpenMemHandle(rank {r})")
            self.bases.append(p.value + self.GUARD)      # the peer's buffer starts behind its front guard
            self._opened.append(p.value)
        self.local_words = torch.zeros(2, dtype=torch.int32, device=device)
        arr = (c_void_p * self.size)(*self.bases)
        self.comm = lib.eredu_comm_create(arr, self.rank, self.size, slot_bytes, out_total, self.local_words.data_ptr())
        if not self.comm:
            raise RuntimeError("eredu_comm_create failed")
        self.out_off = int(lib.eredu_comm_out_offset(self.comm))
        self.out_bytes = (out_bytes + 255) // 256 * 256
        self.x_off = self.out_off + self.out_bytes
        self.x_bytes = x_bytes
        self.slot_bytes = slot_bytes
        self.lam_bytes = (slot_bytes // 2 + 255) // 256 * 256     # per (parity, source) slot of the tag-free one-shot words
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every peer has mapped every buffer before anyone launches a kernel

    GUARD = 4096
    CANARY = 0x5AC3A55A

    def check_canaries(self) -> None:
        """Raises when a store (local or from a peer) landed outside this rank's symmetric buffer."""
        torch.cuda.synchronize(self.device)
        for name, off in (("front", 0), ("back", self.GUARD + self.bytes)):
            g = view_raw(self._alloc + off, (self.GUARD // 4,), torch.int32, self.device)
            bad = int((g != self.CANARY).sum())
            if bad:
                raise RuntimeError(f"peer buffer of rank {self.rank}: {bad} guard words behind the {name} edge were overwritten")

    def out_view(self, shape, dtype) -> torch.Tensor:
        return view_raw(self.own + self.out_off, shape, dtype, self.device)

    def x_view(self, shape, dtype) -> torch.Tensor:
        return view_raw(self.own + self.x_off, shape, dtype, self.device)

    def barrier(self):
        st = native.status_word(self.device)
        native.check(self.lib.eredu_peer_barrier(self.comm, st.data_ptr(), native.stream_ptr(self.device)),
                     "eredu_peer_barrier")

    def close(self):
        if getattr(self, "comm", None):
            torch.cuda.synchronize(self.device)
            self.lib.eredu_comm_destroy(self.comm)
            self.comm = None
            for p in self._opened:
                self.lib.eredu_ipc_close(p)
            self.lib.eredu_peer_free(self._alloc)


class PeerP2P:
    """Point-to-point messages between the ranks of a group over peer memory (``eredu_peer_send`` / ``eredu_peer_recv``):
    kernels on the caller's stream, no host synchronisation, valid inside CUDA-graph capture. Both sides of a channel
    must issue matching calls in the same order; a message is at most ``max_bytes`` (channel 0) or 4 KB (channels 1-3)."""

    CHANNELS = 4

    def __init__(self, group, device: torch.device, max_bytes: int):
        slot = (int(max_bytes) + 4096 * (self.CHANNELS - 1) + 255) // 256 * 256
        self.pg = PeerGroup(group, device, slot, 256)
        self.device = device
        self.rank, self.size = self.pg.rank, self.pg.size
        self.max_bytes = int(max_bytes)
        self.counters = torch.zeros(8 * 2 * self.CHANNELS + 2, dtype=torch.int32, device=device)
        self.sm = torch.cuda.get_device_properties(device).multi_processor_count
        self.lib = native.lib()

    def _args(self, t: torch.Tensor):
        assert t.is_contiguous() and t.device == self.device
        n = t.numel() * t.element_size()
        assert n % 16 == 0, "messages are whole 16-byte words: pad the tensor"
        return t.data_ptr(), n

    def send(self, dst: int, t: torch.Tensor, channel: int = 0) -> None:
        p, n = self._args(t)
        st = native.status_word(self.device)
        native.check(self.lib.eredu_peer_send(self.pg.comm, dst, channel, p, n, self.counters.data_ptr(), self.sm,
                                              st.data_ptr(), native.stream_ptr(self.device)), "eredu_peer_send")

    def recv(self, src: int, out: torch.Tensor, channel: int = 0) -> torch.Tensor:
        p, n = self._args(out)
        st = native.status_word(self.device)
        native.check(self.lib.eredu_peer_recv(self.pg.comm, src, channel, p, n, self.counters.data_ptr(), self.sm,
                                              st.data_ptr(), native.stream_ptr(self.device)), "eredu_peer_recv")
        return out

    def close(self):
        self.pg.close()
