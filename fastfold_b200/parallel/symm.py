"""Symmetric heap over NVLink peer memory and the collectives built on it (csrc/comm_p2p.cu).

``SymmHeap`` allocates one slab per rank of the DAP group with ``torch.distributed._symmetric_memory`` (CUDA VMM
allocation + handle exchange), records every peer's mapped base address, and hands out *slots*: named, fixed
sub-ranges of the slab.  A call site (say "block 17, triangle-multiplication-outgoing right operand") always uses
the same slot, on every rank, so ranks agree on offsets without talking to each other.  Flags and epochs live in a
second, small symmetric allocation.  All data movement is done by this package's own kernels; NCCL is not involved
after the rendezvous, which also makes every collective capturable in a CUDA graph.

Nothing like this exists in the reference, whose collectives are ``torch.distributed`` NCCL calls
(fastfold/distributed/comm.py, comm_async.py).
"""
import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from . import core

MAX_RANKS = 8
MAX_SLOTS = 64
# one-kernel collectives (every rank stores into the destination's slot); FASTFOLD_COMM_PUSH=0 selects publish + pull
PUSH = os.environ.get("FASTFOLD_COMM_PUSH", "1") != "0"
FLAG_WORDS = MAX_SLOTS * 19


class SymmCtx(ctypes.Structure):
    _fields_ = [("heap", ctypes.c_void_p * MAX_RANKS), ("flags", ctypes.c_void_p * MAX_RANKS), ("rank", ctypes.c_int),
                ("world", ctypes.c_int), ("wait_ns", ctypes.c_ulonglong)]


_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_SIG = {
    "ffb_symm_publish": [ctypes.POINTER(SymmCtx), _I, _L, _P, _L, _P],
    "ffb_symm_pull": [ctypes.POINTER(SymmCtx), _I, _L, _P, _L, _I, _P],
    "ffb_symm_a2a_layernorm": [ctypes.POINTER(SymmCtx), _I, _L, _I, _I, _I, _I, _P, _P, _P, _P, _F, _I, _P],
    "ffb_symm_allreduce_bf16": [ctypes.POINTER(SymmCtx), _I, _L, _L, _F, _P],
    "ffb_symm_xchg": [ctypes.POINTER(SymmCtx), _I, _L, _P, _L, _L, _L, _I, _I, _P, _P],
    "ffb_symm_xchg_layernorm": [ctypes.POINTER(SymmCtx), _I, _L, _P, _I, _I, _I, _I, _P, _P, _P, _P, _F, _I, _P],
    "ffb_symm_slot_fence": [ctypes.POINTER(SymmCtx), _I, _I, _P],
    "ffb_symm_consume_fence": [ctypes.POINTER(SymmCtx), _I, _I, _P],
    "ffb_symm_wait_never": [ctypes.POINTER(SymmCtx), _I, _P],
}
_declared = False


def _libc():
    global _declared
    lib = _lib.get()
    if not _declared:
        for name, sig in _SIG.items():
            fn = getattr(lib, name)
            fn.argtypes = sig
            fn.restype = ctypes.c_int
        _declared = True
    return lib


class Slot:
    __slots__ = ("index", "offset", "nbytes", "name")

    def __init__(self, index, offset, nbytes, name):
        self.index, self.offset, self.nbytes, self.name = index, offset, nbytes, name


class SymmHeap:
    """Per-process handle of the symmetric heap of one process group."""

    def __init__(self, group, heap_bytes, wait_s=20.0):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= MAX_RANKS
        dev = torch.device("cuda", torch.cuda.current_device())
        self.heap_bytes = int(heap_bytes + 1023) // 1024 * 1024
        self.heap = symm_mem.empty(self.heap_bytes, dtype=torch.uint8, device=dev)
        self.flags = symm_mem.empty(FLAG_WORDS, dtype=torch.int32, device=dev)
        self.flags.zero_()
        torch.cuda.synchronize()
        self._h_heap = symm_mem.rendezvous(self.heap, group)
        self._h_flags = symm_mem.rendezvous(self.flags, group)
        self.ctx = SymmCtx()
        for r in range(self.world):
            self.ctx.heap[r] = int(self._h_heap.buffer_ptrs[r])
            self.ctx.flags[r] = int(self._h_flags.buffer_ptrs[r])
        self.ctx.rank, self.ctx.world = self.rank, self.world
        self.ctx.wait_ns = int(wait_s * 1e9)
        self.slots = {}
        self._cursor = 0
        self.ring = []
        self._seq = 0
        dist.barrier(group)            # every pad is zeroed before any rank raises a flag in it
        torch.cuda.synchronize()

    def poison(self):
        """Fills this rank's slab with 0xFF bytes (NaN in every floating-point format) - test aid: a consumer that reads
        a peer slot before its producer wrote it, or beyond what was written, then sees NaN instead of stale data."""
        self.heap.fill_(0xFF)
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def make_ring(self, n_slots, slot_bytes):
        """A ring of equally sized slots for the activation collectives; consecutive collectives take consecutive
        slots, so a slot is reused only after ``n_slots - 1`` other exchanges (the flag protocol makes reuse safe)."""
        if not self.ring:
            self.ring = [self.slot("ring%d" % i, slot_bytes) for i in range(n_slots)]
        return self.ring

    def _ensure_ring(self):
        if not self.ring:
            want = _WANT_MESSAGE[0]
            if want:
                # sized from the model's shapes (``request_message_bytes``): every activation collective fits a slot;
                # large slots get a shorter ring (reuse is made safe by the flag protocol, it only costs waiting)
                n = 12 if want <= (256 << 20) else 6
                per = min(want, (self.heap_bytes - self._cursor) // n)
                self.make_ring(n, per // 1024 * 1024)
                return
            per = min(192 << 20, max(1 << 20, (self.heap_bytes - self._cursor) // 2 // 12))
            self.make_ring(12, per)

    def max_message(self):
        """Largest message (bytes) that fits a ring slot; callers send anything larger through NCCL instead."""
        self._ensure_ring()
        return self.ring[0].nbytes

    def next_ring_slot(self, nbytes):
        self._ensure_ring()
        s = self.ring[self._seq % len(self.ring)]
        self._seq += 1
        if nbytes > s.nbytes:
            raise RuntimeError("message of %d bytes exceeds the symmetric ring slot (%d bytes); raise FASTFOLD_SYMM_HEAP_MB" % (nbytes, s.nbytes))
        return s

    # -- slots ------------------------------------------------------------------
    def slot(self, name, nbytes):
        """The slot registered under ``name`` (created on first use; must be requested in the same order on all ranks)."""
        s = self.slots.get(name)
        nbytes = (int(nbytes) + 1023) // 1024 * 1024
        if s is not None:
            if s.nbytes < nbytes:
                raise RuntimeError("symmetric slot %r was created with %d bytes, %d requested" % (name, s.nbytes, nbytes))
            return s
        if len(self.slots) >= MAX_SLOTS:
            raise RuntimeError("out of symmetric slots (%d)" % MAX_SLOTS)
        if self._cursor + nbytes > self.heap_bytes:
            raise RuntimeError("symmetric heap exhausted: %d + %d > %d" % (self._cursor, nbytes, self.heap_bytes))
        s = Slot(len(self.slots), self._cursor, nbytes, name)
        self._cursor += nbytes
        self.slots[name] = s
        return s

    def view(self, slot, shape, dtype, rank=None):
        """Tensor view of a slot in this rank's slab (``rank=None``) - peers' slabs are only touched by kernels."""
        n = 1
        for d in shape:
            n *= d
        nb = n * torch.empty((), dtype=dtype).element_size()
        assert nb <= slot.nbytes
        return self.heap[slot.offset:slot.offset + nb].view(dtype).view(shape)

    # -- raw collectives ----------------------------------------------------------
    def publish(self, slot, src):
        src = src.contiguous()
        nb = src.numel() * src.element_size()
        assert nb % 16 == 0 and nb <= slot.nbytes
        _lib.check(_libc().ffb_symm_publish(ctypes.byref(self.ctx), slot.index, slot.offset, _lib.ptr(src), nb, _lib.stream_ptr()), "symm_publish")
        return nb

    def pull(self, slot, dst, bytes_per_rank, all_to_all):
        _lib.check(_libc().ffb_symm_pull(ctypes.byref(self.ctx), slot.index, slot.offset, _lib.ptr(dst), bytes_per_rank, 1 if all_to_all else 0,
                                         _lib.stream_ptr()), "symm_pull")

    # -- one-kernel ("push") collectives -------------------------------------------------------------------
    def fits_push(self, chunk_bytes):
        """True when a push collective whose per-source-rank share is ``chunk_bytes`` fits a ring slot (the slot receives
        one share from every rank) and the share is a whole number of 16-byte units."""
        return PUSH and chunk_bytes % 16 == 0 and 0 < chunk_bytes * self.world <= self.max_message()

    def _xchg(self, name, src, x1, x2, chunk_bytes, scatter, mode, out):
        s = self.next_ring_slot(chunk_bytes * self.world) if name is None else self.slot(name, chunk_bytes * self.world)
        _lib.check(_libc().ffb_symm_xchg(ctypes.byref(self.ctx), s.index, s.offset, _lib.ptr(src), x1, x2, chunk_bytes, 1 if scatter else 0, mode,
                                         _lib.ptr(out), _lib.stream_ptr()), "symm_xchg")
        return out

    def gather_dim(self, x, dim, name=None):
        """All-gather of ``x`` along ``dim`` in ONE kernel: every rank stores its shard into every rank's slot, waits
        for the others' shards and copies them into the result already concatenated along ``dim``."""
        x = x.contiguous()
        dim = dim % x.dim()
        nb = x.numel() * x.element_size()
        lead = 1
        for d in x.shape[:dim]:
            lead *= d
        shape = list(x.shape)
        shape[dim] *= self.world
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
        return self._xchg(name, x, 1, lead, nb, False, 1 if lead > 1 else 0, out)

    def all_to_all_dims(self, x, in_dim, out_dim, name=None):
        """Splits ``in_dim`` of ``x`` over the ranks and concatenates what arrives along ``out_dim``, in ONE kernel."""
        x = x.contiguous()
        in_dim, out_dim = in_dim % x.dim(), out_dim % x.dim()
        P = self.world
        shape = list(x.shape)
        shape[in_dim] //= P
        x1 = 1
        for d in x.shape[:in_dim]:
            x1 *= d
        x2 = 1
        for d in shape[:out_dim]:
            x2 *= d
        chunk = x.numel() * x.element_size() // P
        oshape = list(shape)
        oshape[out_dim] *= P
        out = torch.empty(oshape, dtype=x.dtype, device=x.device)
        return self._xchg(name, x, x1, x2, chunk, True, 1 if x2 > 1 else 0, out)

    def reduce_scatter_dim(self, x, dim, name=None):
        """Sum over the ranks, keep this rank's slice along ``dim`` (bf16 in / out, fp32 accumulation), in ONE kernel:
        slice q of every rank is stored into rank q's slot and summed there."""
        x = x.contiguous()
        dim = dim % x.dim()
        P = self.world
        shape = list(x.shape)
        shape[dim] //= P
        x1 = 1
        for d in x.shape[:dim]:
            x1 *= d
        chunk = x.numel() * x.element_size() // P
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
        return self._xchg(name, x, x1, 1, chunk, True, 2, out)

    def all_gather(self, name, x):
        """Stacks ``x`` of every rank along a new leading dimension: ``[P, *x.shape]``."""
        x = x.contiguous()
        nb = x.numel() * x.element_size()
        if self.fits_push(nb):
            out = torch.empty((self.world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
            return self._xchg(name, x, 1, 1, nb, False, 0, out)
        s = self.next_ring_slot(nb) if name is None else self.slot(name, nb)
        self.publish(s, x)
        out = torch.empty((self.world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        self.pull(s, out, nb, False)
        return out

    def all_to_all(self, name, send):
        """``send [P, ...]``: chunk q goes to rank q; returns ``recv [P, ...]`` with chunk r coming from rank r."""
        send = send.contiguous()
        nb = send.numel() * send.element_size()
        if self.fits_push(nb // self.world):
            return self._xchg(name, send, 1, 1, nb // self.world, True, 0, torch.empty_like(send))
        s = self.next_ring_slot(nb) if name is None else self.slot(name, nb)
        self.publish(s, send)
        recv = torch.empty_like(send)
        self.pull(s, recv, nb // self.world, True)
        return recv

    def a2a_layer_norm(self, name, x, mode, A, B, C, gamma, beta, eps, want_raw=True, transpose_norm=False):
        """Axis switch of the shard ``x`` fused with LayerNorm: one kernel that stores the shard's rows into the
        destination ranks' slots and normalises what arrives (csrc/comm_p2p.cu ``symm_xchg_ln_k``); the two-kernel
        publish + pull form (``symm_a2a_ln_k``) remains for ``FASTFOLD_COMM_PUSH=0``."""
        x = x.contiguous()
        nb = x.numel() * x.element_size()
        P = self.world
        Ad, Bd = (A, B // P) if mode == 0 else (A // P, B)
        raw = torch.empty(Ad, Bd, C, dtype=x.dtype, device=x.device) if want_raw else None
        norm = None
        if gamma is not None:
            norm = torch.empty((Bd, Ad, C) if transpose_norm else (Ad, Bd, C), dtype=x.dtype, device=x.device)
        s = self.next_ring_slot(nb) if name is None else self.slot(name, nb)
        if PUSH:
            _lib.check(_libc().ffb_symm_xchg_layernorm(ctypes.byref(self.ctx), s.index, s.offset, _lib.ptr(x), mode, A, B, C, _lib.ptr(raw),
                                                       _lib.ptr(norm), _lib.ptr(gamma), _lib.ptr(beta), float(eps), 1 if transpose_norm else 0,
                                                       _lib.stream_ptr()), "symm_xchg_layernorm")
            return raw, norm
        self.publish(s, x)
        _lib.check(_libc().ffb_symm_a2a_layernorm(ctypes.byref(self.ctx), s.index, s.offset, mode, A, B, C, _lib.ptr(raw), _lib.ptr(norm),
                                                  _lib.ptr(gamma), _lib.ptr(beta), float(eps), 1 if transpose_norm else 0, _lib.stream_ptr()),
                   "symm_a2a_layernorm")
        return raw, norm

    def all_reduce_(self, name_or_slot, n_elems, scale=1.0):
        """In-place sum over ranks of the bf16 vector stored in the slot (e.g. the flat gradient buffer)."""
        s = name_or_slot if isinstance(name_or_slot, Slot) else self.slots[name_or_slot]
        _lib.check(_libc().ffb_symm_allreduce_bf16(ctypes.byref(self.ctx), s.index, s.offset, n_elems, float(scale), _lib.stream_ptr()),
                   "symm_allreduce_bf16")

    # -- producer / consumer fences for kernels that write or read a slot themselves ----------------------
    def slot_fence(self, slot, pre):
        """``pre=True`` (before the producer kernel): wait until every peer has finished with the slot's previous
        contents.  ``pre=False`` (after it): raise this rank's ready flag on every peer."""
        _lib.check(_libc().ffb_symm_slot_fence(ctypes.byref(self.ctx), slot.index, 1 if pre else 0, _lib.stream_ptr()), "symm_slot_fence")

    def consume_fence(self, slot, pre):
        """``pre=True`` (before a kernel that reads peers' slots): wait for every peer's ready flag.  ``pre=False``
        (after it): raise this rank's done flag on every peer and advance the slot's epoch."""
        _lib.check(_libc().ffb_symm_consume_fence(ctypes.byref(self.ctx), slot.index, 1 if pre else 0, _lib.stream_ptr()), "symm_consume_fence")

    def peer_addresses(self, slot, byte_offset=0):
        """Address of ``slot`` (+ offset) in every rank's slab, as mapped on this GPU."""
        return [int(self.ctx.heap[r]) + slot.offset + byte_offset for r in range(self.world)]

    def wait_never(self, slot):
        """Test hook: a kernel waits for a flag nobody raises; returns after the heap's wait limit with status 4."""
        _lib.check(_libc().ffb_symm_wait_never(ctypes.byref(self.ctx), slot.index, _lib.stream_ptr()), "symm_wait_never")


_HEAPS = {}
_WANT_MESSAGE = [0]


def request_message_bytes(nbytes):
    """Tells the heap, before it is created, how large the largest activation collective of the coming run is (per
    rank); the heap is then sized so that a ring slot holds it and nothing falls back to NCCL.  ``ring_bytes_for`` gives
    the number for a model call."""
    _WANT_MESSAGE[0] = max(_WANT_MESSAGE[0], (int(nbytes) + 1023) // 1024 * 1024)


def ring_bytes_for(n_res, n_seq, n_extra, world, c_z=128, c_m=256, c_e=64, elem=2):
    """Largest per-rank message of one model call over ``world`` DAP ranks: the pair shard's axis switch, the MSA / extra
    MSA shards, and the slot a rank's projected triangle-multiplication operands (both, channel-major) are written to
    for the peers' GEMMs to read."""
    if world <= 1:
        return 0
    pad = (-n_res) % world
    n = n_res + pad
    z_shard = n * n // world * c_z * elem
    return max(2 * z_shard, n_seq * n // world * c_m * elem * 2, n_extra * n // world * c_e * elem * 2)


def get_heap(kind="dap", heap_bytes=None, wait_s=None):
    """The symmetric heap of the DAP group (``kind='dap'``) or of the whole world (``kind='world'``); None when the
    group has one rank, when there is no GPU, or when ``FASTFOLD_COMM=nccl`` selects the NCCL baseline."""
    if not torch.cuda.is_available() or os.environ.get("FASTFOLD_COMM", "p2p") == "nccl":
        return None
    m = core.mesh()
    if kind == "dap":
        if m.dap_size <= 1:
            return None
        group = m.dap_group
    else:
        if m.world_size <= 1:
            return None
        group = dist.group.WORLD
    h = _HEAPS.get(kind)
    if h is None:
        if kind == "world" and m.dap_size == m.world_size and "dap" in _HEAPS:
            h = _HEAPS["dap"]
        elif kind == "dap" and m.dap_size == m.world_size and "world" in _HEAPS:
            h = _HEAPS["world"]
        else:
            nbytes = heap_bytes or int(os.environ.get("FASTFOLD_SYMM_HEAP_MB", "2048")) * (1 << 20)
            if _WANT_MESSAGE[0]:
                n = 12 if _WANT_MESSAGE[0] <= (256 << 20) else 6
                nbytes = max(nbytes, n * _WANT_MESSAGE[0] + (512 << 20))
            h = SymmHeap(group, nbytes, wait_s=wait_s if wait_s is not None else float(os.environ.get("FASTFOLD_SYMM_WAIT_S", "20")))
        _HEAPS[kind] = h
    return h


def release_all():
    _HEAPS.clear()
