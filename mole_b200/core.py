"""Host-side orchestrator of the expert pipeline -- the Python face of what the reference
bound as the ``core`` extension (MOLE/cpp/core.cpp:1347-1469).

``create_UniMem``        the GPU slot pool for offloaded experts (MOLE/cpp/umemory.cpp:77-86)
``MOLECore``             per-layer object: parameter cores, prefetch, and the forward /
                         backward pipelines of ``_BatchFusedFWD`` (MOLE/cpp/core.cpp:991-1131,
                         1133-1300) over "records" of at most ``ebatch_size`` experts.

The pipeline keeps the reference's three phases per group of records -- exchange + parameter
fetch, expert compute, return exchange -- on the communication / transfer / compute streams,
but every phase is a call into ``libmole_b200.so`` on capacity-strided rows: no per-record
tensor allocation, no permute/contiguous re-layout (core.cpp:233, 240) and no re-assembly
copies (core.cpp:1097-1124); the grouped GEMM reads the (source rank, expert) chunks where
the exchange put them and the return exchange writes straight into the output tensor.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import ops
from ._lib import check, lib
from .utils.Udist import MOLEDist
from .utils.Ustream import ExpertStreamCtx


# --------------------------------------------------------------------------- #
# slot pool ("UniMem")
# --------------------------------------------------------------------------- #
class UniMem:
    """``pool_size`` expert slots for each of W1 ``[F, M]``, b1 ``[F]``, W2 ``[F, M]``, b2 ``[M]``."""
    _instance: Optional["UniMem"] = None

    def __init__(self, device: int, pool_size: int, dtype: torch.dtype, sizes, dry: bool = False):
        self.device = device
        self.pool_size = pool_size
        self.dtype = dtype
        self.sizes = [list(s) for s in sizes]
        self.handle = None
        self.bases: List[Optional[torch.Tensor]] = [None] * 4
        if pool_size == -1:
            return
        F, M = self.sizes[0]
        handle = C.c_void_p()
        ctx = None if dry else ExpertStreamCtx.get(torch.device("cuda", device)).handle
        check(lib.mole_pool_create(ctx, pool_size, M, F, ops._DTYPES[dtype], C.byref(handle)))
        self.handle = handle
        self.dry = dry
        self.bases = [self.base_ptr(i) for i in range(4)]

    # -- thin wrappers -----------------------------------------------------------------
    def base_ptr(self, p_id: int) -> int:
        p = C.c_void_p()
        check(lib.mole_pool_base(self.handle, p_id, C.byref(p)))
        return p.value or 0

    def view_pool_size(self) -> int:
        n = C.c_int32()
        check(lib.mole_pool_view_size(self.handle, C.byref(n)))
        return n.value

    def clear_virtual_mem(self) -> None:
        check(lib.mole_pool_clear_virtual(self.handle))

    def prefetch(self, moe_id: int, n: int) -> int:
        first = C.c_int32()
        check(lib.mole_pool_prefetch(self.handle, moe_id, n, C.byref(first)))
        return first.value

    def fetch_top_prefetched_batch(self, moe_id: int) -> int:
        n = C.c_int32()
        check(lib.mole_pool_pop_prefetched(self.handle, moe_id, C.byref(n)))
        return n.value

    def fetch(self, host_params, e0: int, n: int, slot0: int, skip: int,
              absolute: bool = False) -> int:
        arr = (C.c_void_p * 4)(*[t.data_ptr() if t is not None else None for t in host_params])
        ticket = C.c_int32()
        check(lib.mole_pool_fetch(self.handle, arr, e0, n, slot0, skip, int(absolute),
                                  C.byref(ticket)))
        return ticket.value

    def wait_fetch(self, ticket: int, stream: torch.cuda.Stream) -> None:
        check(lib.mole_pool_wait_fetch(self.handle, ticket, C.c_void_p(stream.cuda_stream)))

    def mark_used(self, slot0: int, n: int, stream: torch.cuda.Stream) -> None:
        check(lib.mole_pool_mark_used(self.handle, slot0, n, C.c_void_p(stream.cuda_stream)))

    def abs_slot(self, view_slot: int) -> int:
        a = C.c_int32()
        check(lib.mole_pool_abs_slot(self.handle, view_slot, C.byref(a)))
        return a.value

    def log(self):
        n = C.c_int32()
        check(lib.mole_pool_log(self.handle, None, 0, C.byref(n)))
        buf = (C.c_int32 * (4 * max(n.value, 1)))()
        check(lib.mole_pool_log(self.handle, buf, n.value, C.byref(n)))
        return [tuple(buf[4 * i:4 * i + 4]) for i in range(n.value)]


def create_UniMem(device: int, pool_size: int, dtype, sizes, dry: bool = False) -> UniMem:
    """One pool per process, shared by all layers (MOLE/cpp/umemory.cpp:77-86)."""
    if isinstance(dtype, str):
        dtype = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16}[dtype]
    if UniMem._instance is None:
        UniMem._instance = UniMem(device, pool_size, dtype, sizes, dry)
    return UniMem._instance


def _get_UniMem() -> UniMem:
    return UniMem._instance


def clear_virtual_mem() -> None:
    """Drops every prefetch reservation of the pool (``clear_virtual_mem`` of the reference's
    ``core`` module; the scheduler calls it at the start of a step)."""
    if UniMem._instance is not None and UniMem._instance.handle is not None:
        UniMem._instance.clear_virtual_mem()


def fast_assign_prefetch(P: int, F, E):
    """``(GPscheme, LPscheme)`` as the reference's binding returns them
    (MOLE/cpp/core.cpp:1302-1345): ``LPscheme[i]`` experts layer ``i`` prefetches for itself,
    ``GPscheme[i]`` a list of ``[layer j, count]``: while layer ``i`` runs it also fetches ``count``
    experts of the later layer ``j`` into spare pool slots."""
    n = len(E)
    assert len(F) == n
    Fa = (C.c_int32 * max(n, 1))(*F)
    Ea = (C.c_int32 * max(n, 1))(*E)
    local = (C.c_int32 * max(n, 1))()
    cap = 4 * max(n, 1) + 8
    while True:
        triples = (C.c_int32 * (3 * cap))()
        nt = C.c_int32()
        check(lib.mole_fast_assign_prefetch(P, Fa, Ea, n, local, triples, cap, C.byref(nt)))
        if nt.value <= cap:
            break
        cap = nt.value
    gp = [[] for _ in range(n)]
    for j in range(nt.value):
        gp[triples[3 * j]].append([triples[3 * j + 1], triples[3 * j + 2]])
    return gp, [local[i] for i in range(n)]


# --------------------------------------------------------------------------- #
# records
# --------------------------------------------------------------------------- #
@dataclass
class Record:
    """A batch of consecutive local experts processed by one FFN call
    (``_BatchRecord``, MOLE/cpp/define.hpp:613-677)."""
    use_cpu_param: bool
    batch_base: int       # first expert inside its kind (GPU-resident or offloaded)
    base_in_all: int      # first local expert index
    batch_size: int
    prefetched: int = 0   # leading experts already in their slots
    view_base: int = 0    # first pool slot (view coordinates)
    ticket: int = -1      # pool fetch ticket
    slots: List[int] = field(default_factory=list)


class _DeviceBytes:
    """Raw device memory as a ``__cuda_array_interface__`` object (so that torch can view it)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class PeerExchange:
    """Receive buffers of the push-style exchange of one layer, visible to every rank of the node.

    Instead of filling a local buffer and sending it (``first_a2a`` / ``second_a2a``,
    MOLE/cpp/core.cpp:144-210), the producing kernel stores each row straight into the memory of
    the rank that consumes it, over NVLink:

      x0   [W, L, Cs, M]   dispatch rows for my experts        written by every rank's dispatch
      ret  [E, Cs, M]      expert outputs for my tokens        written by the owners' FC2 epilogue
      g    [W, L, Cs, M]   output gradients for my experts     written by every rank's combine bwd
      dx   [E, Cs, M]      input gradients for my tokens       written by the owners' dX epilogue
      counts [W * L] i32   valid rows per (source, expert)     written with the dispatch rows

    Each buffer is plain device memory exported through a CUDA IPC handle and mapped by the peers
    (no multicast object).  Writers and readers are ordered by four barriers per fwd+bwd
    (``mole_barrier``): every reader of a buffer has finished before the barrier that precedes
    its next writer, see ``MOLECore.forward_peer`` / ``backward_peer``."""

    KINDS = ("x0", "ret", "g", "dx", "counts", "flags", "allcounts")
    BARRIER_LIMIT_NS = 2_000_000_000      # a rank that never arrives costs its peers two seconds

    def __init__(self, world, rank, L, Cs, M, dtype, device, group):
        import torch.distributed as dist
        self.world, self.rank, self.L, self.M, self.dtype = world, rank, L, M, dtype
        self.device, self.group = device, group
        self.cap_Cs = Cs         # rows per chunk the buffers hold; smaller strides reuse them
        self.key = (world, L, M, dtype)
        es = torch.empty(0, dtype=dtype).element_size()
        row_bytes = world * L * Cs * M * es
        sizes = {"x0": row_bytes, "ret": row_bytes, "g": row_bytes, "dx": row_bytes,
                 "counts": max(256, world * L * 4), "flags": 256,
                 "allcounts": max(256, world * world * L * 4)}
        self.sizes = sizes
        # Every rank takes the same decision: each phase ends in a collective that carries the
        # ranks' success flags, and one failure anywhere makes all of them give the buffers up
        # (the caller then uses the all-to-all pipeline on every rank).
        self.own, self.mapped, self.table = {}, [], {}
        handles, err = [], None
        try:
            for kind in self.KINDS:
                p = C.c_void_p()
                check(lib.mole_peer_alloc(sizes[kind], C.byref(p)))
                self.own[kind] = p.value
                h = (C.c_uint8 * 64)()
                check(lib.mole_peer_export(p, h))
                handles.append(bytes(h))
        except Exception as e:
            err = e
            handles = [bytes(64)] * len(self.KINDS)
        blob = b"".join(handles) + bytes([0 if err else 1])
        mine = torch.tensor(list(blob), dtype=torch.uint8, device=device)
        every = torch.empty(world * mine.numel(), dtype=torch.uint8, device=device)
        dist.all_gather_into_tensor(every, mine, group=group)
        every = every.cpu().view(world, -1)
        if int(every[:, -1].min()) == 0:
            self.close()
            raise RuntimeError(f"peer buffers could not be allocated or exported on every rank ({err})")
        every = every[:, :-1].reshape(world, len(self.KINDS), 64)
        try:
            for ki, kind in enumerate(self.KINDS):
                ptrs = []
                for q in range(world):
                    if q == rank:
                        ptrs.append(self.own[kind])
                        continue
                    h = (C.c_uint8 * 64)(*every[q, ki].tolist())
                    p = C.c_void_p()
                    check(lib.mole_peer_open(h, C.byref(p)))
                    self.mapped.append(p.value)
                    ptrs.append(p.value)
                self.table[kind] = (C.c_void_p * world)(*ptrs)
        except Exception as e:
            err = e
        flag = torch.tensor([0 if err else 1], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            self.close(True, group)
            raise RuntimeError(f"peer buffers could not be mapped on every rank ({err})")
        self.Cs = None
        self.set_stride(Cs)
        self.scratch = torch.zeros(8 * world, dtype=torch.uint8, device=device)
        self.barrier_seq = 0     # flag barriers taken so far (the same number on every rank)
        import os
        self.flag_barrier = os.environ.get("MOLE_FLAG_BARRIER", "1") != "0"
        # packed: every rank first learns every rank's counts, then stores its rows at their
        # final place in the owner's per-expert run; the owner gathers nothing
        # (MOLE_PACKED_PUSH=0: chunks per source rank, packed by the owner before its GEMMs)
        self.packed = os.environ.get("MOLE_PACKED_PUSH", "1") != "0"
        self.serial = 0          # forward passes so far: backward checks that its buffers are still its own
        dist.barrier(group=group)

    def set_stride(self, Cs: int) -> None:
        """Views of the buffers for chunks of ``Cs <= cap_Cs`` rows (a shorter batch, another
        capacity factor): the same memory with a smaller stride, nothing is reallocated."""
        if Cs == self.Cs:
            return
        assert Cs <= self.cap_Cs
        world, L, M, dtype = self.world, self.L, self.M, self.dtype

        def view(kind, tdtype, shape):
            mem = _DeviceBytes(self.own[kind], self.sizes[kind])
            t = torch.as_tensor(mem, device=self.device)
            n = 1
            for s in shape:
                n *= s
            return t[: n * torch.empty(0, dtype=tdtype).element_size()].view(tdtype).view(*shape)

        E = world * L
        self.Cs = Cs
        # chunks [W][L][Cs] or, packed, one run per local expert [L][W * Cs]: the same memory
        self.x0 = view("x0", dtype, (world, L, Cs, M))
        self.g = view("g", dtype, (world, L, Cs, M))
        self.allcounts = view("allcounts", torch.int32, (world, world * L))
        self.ret = view("ret", dtype, (E, Cs, M))
        self.dx = view("dx", dtype, (E, Cs, M))
        self.counts = view("counts", torch.int32, (world * L,))

    def barrier(self):
        """Every rank has finished what it enqueued so far on the current stream: flags stored
        into the peers' mapped memory with a bounded wait (``MOLE_FLAG_BARRIER=0``: a 4-byte
        grouped NCCL send/recv instead)."""
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        if self.flag_barrier:
            self.barrier_seq += 1
            check(lib.mole_peer_barrier(self.table["flags"], self.world, self.rank, self.barrier_seq,
                                        self.BARRIER_LIMIT_NS, stream))
        else:
            check(lib.mole_barrier(MOLEDist._instance.comm, C.c_void_p(self.scratch.data_ptr()), stream))

    def close(self, barrier=False, group=None):
        """Unmaps the peers' buffers, then frees this rank's own.  ``barrier=True`` (then every
        rank must call it) puts a barrier between the two: a mapping has to be closed before its
        owner frees the memory."""
        for p in self.mapped:
            lib.mole_peer_close(C.c_void_p(p))
        self.mapped = []
        if barrier:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=group)
        for p in self.own.values():
            lib.mole_peer_free(C.c_void_p(p))
        self.own = {}
        for name in ("x0", "g", "ret", "dx", "counts", "allcounts"):
            self.__dict__.pop(name, None)

    def __del__(self):
        # Last resort (interpreter exit, a layer dropped without teardown): no collective is
        # possible here, so only this process's mappings and memory are released.  The peers'
        # mappings of this memory stay valid for them until they close them (CUDA IPC keeps the
        # allocation alive while it is mapped elsewhere).
        try:
            self.close()
        except Exception:
            pass


def exchange_geometry(rec: "Record", local_experts: int, chunk_bytes: int):
    """Byte geometry of one record's all-to-all inside the ``[W][L][Cs][M]`` chunk buffers:
    ``(bytes_per_peer, peer_stride_bytes, byte_offset)``.  Peer ``q``'s block starts at
    ``q * L * chunk``; the record covers its experts ``[base_in_all, base_in_all + batch_size)``
    of every block (MOLE/cpp/core.cpp:144-179 addresses the same sub-blocks per expert batch)."""
    return (rec.batch_size * chunk_bytes, local_experts * chunk_bytes, rec.base_in_all * chunk_bytes)


def build_records(s_experts: int, d_experts: int, ebatch_size: int, use_pool: bool,
                  view_pool_size: int, prefetched: int):
    """Records and launch groups exactly as MOLE/cpp/core.cpp:1009-1051 builds them: GPU-resident
    experts in steps of ``ebatch_size``; offloaded experts in steps of
    ``min(ebatch_size, visible pool)``, a new group whenever the pool wraps."""
    records: List[Record] = []
    groups: List[List[int]] = []
    cur: List[int] = []
    for i in range(0, s_experts, ebatch_size):
        size = min(ebatch_size, s_experts - i)
        cur.append(len(records))
        records.append(Record(False, i, i, size))
    d_batch = min(ebatch_size, view_pool_size if use_pool else 10000)
    if d_experts > 0 and d_batch < 1:
        raise RuntimeError("no pool slot is visible for the offloaded experts")
    view_base = 0
    for i in range(0, d_experts, max(d_batch, 1)):
        size = min(d_batch, d_experts - i)
        if use_pool and view_pool_size - view_base < size:
            view_base = 0
            groups.append(cur)
            cur = []
        cur.append(len(records))
        cur_pref = min(size, prefetched - i) if prefetched > i else 0
        records.append(Record(True, i, i + s_experts, size, cur_pref, view_base))
        view_base += size
    if cur:
        groups.append(cur)
    return records, groups


# --------------------------------------------------------------------------- #
# per-layer core
# --------------------------------------------------------------------------- #
class _Saved:
    """Activations one forward keeps for its backward (``x0`` and ``extras[0]`` of the
    reference's records, MOLE/cpp/define.hpp:638-639)."""
    __slots__ = ("x0", "x1", "h", "counts", "Cs", "n_src", "serial")


class _Staging:
    """One record's worth of device memory for an offloaded batch's backward: the four weight
    gradients and, when the optimizer step runs on the GPU, the Adam moments (and the host's
    accumulated gradient).  ``busy`` is recorded on the device-to-host stream behind the last
    copy that reads the block; the next writer waits for it."""

    def __init__(self, n, M, F, dtype, device):
        kw = dict(dtype=dtype, device=device)
        self.shapes = [(n, F, M), (n, F), (n, F, M), (n, M)]
        self.kw = kw
        self.grads = [torch.empty(*sh, **kw) for sh in self.shapes]
        self.m = self.v = self.g_host = None
        self.busy = None

    def ensure_moments(self, extra_grad: bool) -> None:
        if self.m is None:
            self.m = [torch.empty(*sh, **self.kw) for sh in self.shapes]
            self.v = [torch.empty(*sh, **self.kw) for sh in self.shapes]
        if extra_grad and self.g_host is None:
            self.g_host = [torch.empty(*sh, **self.kw) for sh in self.shapes]

    def acquire(self, stream) -> None:
        if self.busy is not None:
            ExpertStreamCtx.wait_ticket(stream, self.busy)

    def release(self, back_stream) -> None:
        self.busy = ExpertStreamCtx.record(back_stream)


class MOLECore:
    def __init__(self, use_pool, grad_use_pool, mome_use_pool, vari_use_pool, s_experts, d_experts,
                 ebatch_size, world_size, act, adv_adam, acc_step, step, device, moe_id,
                 total_experts, *, dtype=torch.float32, gelu_bwd="exact", ffn_backend=0):
        self.use_pool = bool(use_pool)
        self.grad_use_pool, self.mome_use_pool, self.vari_use_pool = grad_use_pool, mome_use_pool, vari_use_pool
        self.s_experts, self.d_experts = s_experts, d_experts
        self.ebatch_size = max(1, ebatch_size)
        self.world_size = world_size
        self.act_name = act
        self.adv_adam = adv_adam
        self.acc_step = acc_step
        self.step = step
        self.device = device
        self.moe_id = moe_id
        self.total_experts = total_experts
        self.dtype = dtype
        self.gelu_bwd = gelu_bwd
        self.ffn_backend = ffn_backend
        self.fwd_base = 0
        self.bwd_base = 0
        self.gpu_params = [None] * 4
        self.gpu_grads = [None] * 4
        self.cpu_params = [None] * 4
        self.cpu_grads = [None] * 4
        self.cpu_mome = [None] * 4
        self.cpu_vari = [None] * 4
        self._saved: Optional[_Saved] = None
        self._records: List[Record] = []
        self._staging: List["_Staging"] = []
        self._staging_turn = 0
        self._pending_acc = []
        self._peer: Optional[PeerExchange] = None
        self._peer_failed = False
        # Adam hyper-parameters of the step fused behind backward (``set_adam``); ``t`` counts the
        # optimizer steps already taken.  ``hybrid_adam_count`` experts (from the front of the
        # offloaded ones) are updated on the GPU, the rest by the host optimizer.
        self.adam = dict(beta1=0.9, beta2=0.999, t=0, lr=1e-3, lam=0.0, eps=1e-8, adamW=False)
        self.hybrid_adam_count = d_experts

    # -- parameter cores (MOLE/cpp/uparameter.cpp:13-56) -----------------------------------
    def set_GPUParamCore(self, p_id, all_tensors, grad_tensors, bias):
        self.gpu_params[p_id], self.gpu_grads[p_id] = all_tensors, grad_tensors

    def set_CPUParamCore(self, p_id, t, grad, mome, vari, bias, p_id2=None):
        self.cpu_params[p_id], self.cpu_grads[p_id] = t, grad
        self.cpu_mome[p_id], self.cpu_vari[p_id] = mome, vari

    def set_adam(self, beta1, beta2, t, lr, lam, eps, adamW, hybrid_adam_count):
        """Hyper-parameters of the GPU Adam step for offloaded experts
        (``_MOLECore::set_adam``, MOLE/cpp/define.hpp:524-541); ``hybrid_adam_count == -1`` means
        all of them."""
        self.adam = dict(beta1=float(beta1), beta2=float(beta2), t=int(t), lr=float(lr),
                         lam=float(lam), eps=float(eps), adamW=bool(adamW))
        self.hybrid_adam_count = self.d_experts if hybrid_adam_count == -1 else int(hybrid_adam_count)

    def clear_tran_tmp(self):
        """The reference frees temporaries of its D2H callbacks here (MOLE/cpp/define.hpp:366-378);
        this pipeline has none: its staging blocks are guarded by events."""

    def GPUParamCore_fetch_single(self, p_id, i):
        return self.gpu_params[p_id][i]

    def GPUParamCore_fetch_single_grad(self, p_id, i):
        return self.gpu_grads[p_id][i]

    def CPUParamCore_fetch_single(self, p_id, i):
        return self.cpu_params[p_id][i]

    def CPUParamCore_fetch_single_grad(self, p_id, i):
        return self.cpu_grads[p_id][i]

    def set_lazy_zero(self):
        for g in self.cpu_grads:
            if g is not None:
                g.lazy_zero = True

    def unset_lazy_zero(self):
        for g in self.cpu_grads:
            if g is not None:
                g.lazy_zero = False

    # -- prefetch (MOLE/cpp/core.cpp:25-75) ------------------------------------------------
    def _prefetch(self, base_attr: str, batch_size: int) -> None:
        if batch_size == 0 or self.d_experts == 0:
            return
        pool = _get_UniMem()
        base = getattr(self, base_attr)
        batch_size = min(batch_size, self.d_experts - base)
        if batch_size <= 0:
            return
        first = pool.prefetch(self.moe_id, batch_size)
        pool.fetch(self.cpu_params, base, batch_size, first, 0, absolute=True)
        setattr(self, base_attr, base + batch_size)

    def prefetch_fwd(self, batch_size: int) -> None:
        self._prefetch("fwd_base", batch_size)

    def prefetch_bwd(self, batch_size: int) -> None:
        self._prefetch("bwd_base", batch_size)

    def dummy_fetch(self, batch_size: int) -> None:
        if batch_size == 0:
            return
        _get_UniMem().fetch(self.cpu_params, 0, batch_size, 0, 0)

    # -- push-style exchange ---------------------------------------------------------------
    def peer_for(self, Cs: int, M: int, dtype, device) -> Optional[PeerExchange]:
        """The layer's ``PeerExchange`` when the exchange can be pushed (several ranks of one
        node, GPU-resident experts in one record, the bf16 tensor-core path), else ``None`` and
        the pipeline uses the all-to-all.  ``MOLE_PEER_EXCHANGE=0`` switches it off."""
        import os
        W = self.world_size
        L = self.s_experts + self.d_experts
        if (W < 2 or W > 16 or self.d_experts > 0 or self.ebatch_size < L or self._peer_failed
                or dtype != torch.bfloat16 or self.ffn_backend == 1
                or os.environ.get("MOLE_PEER_EXCHANGE", "1") == "0"
                or MOLEDist._instance is None or MOLEDist._instance.comm is None):
            return None
        F = self._ffn_dim()
        if M % 128 or F % 128:
            return None
        key = (W, L, M, dtype)
        peer = self._peer
        if peer is not None and peer.key == key and Cs <= peer.cap_Cs:
            peer.set_stride(Cs)          # shorter batch / other capacity factor: same memory
            return peer
        # First use, or the chunks have outgrown the buffers.  Every rank takes this branch in the
        # same call: the token count per rank (hence Cs) must be equal on all ranks, as the
        # reference's equal-split exchange requires too (MOLE/cpp/core.cpp:156-161).  The old
        # buffers go first, collectively: unmap everywhere, barrier, then free.
        if peer is not None:
            peer.close(True, MOLEDist._instance.MOLE_group)
            self._peer = None
        try:
            self._peer = PeerExchange(W, MOLEDist._instance.rank, L, Cs, M, dtype, device,
                                      MOLEDist._instance.MOLE_group)
        except Exception as e:      # no peer mapping on this system: keep the all-to-all
            import warnings
            warnings.warn(f"push-style exchange unavailable ({e}); using the all-to-all")
            self._peer_failed = True
            self._peer = None
        return self._peer

    def close_peer_exchange(self) -> None:
        """Collective teardown of the layer's push-exchange buffers (every rank calls it)."""
        if self._peer is not None:
            self._peer.close(True, MOLEDist._instance.MOLE_group)
            self._peer = None

    def forward_peer(self, peer: PeerExchange, requires_grad: bool) -> torch.Tensor:
        """Expert pipeline when the dispatch has already pushed this rank's rows into the owners'
        ``x0`` buffers: barrier, grouped FFN whose FC2 epilogue stores the outputs into the
        source ranks' ``ret`` buffers, barrier.  Returns this rank's ``ret`` ``[E, Cs, M]``."""
        self._check_fault()
        W, L, Cs, M = peer.world, peer.L, peer.Cs, peer.M
        F = self._ffn_dim()
        records, _ = build_records(self.s_experts, 0, self.ebatch_size, False, 0, 0)
        rec = records[0]
        peer.serial += 1
        peer.barrier()                      # every rank's dispatch rows and counts have landed
        rows_total = W * L * Cs
        x1 = torch.empty(rows_total, F, dtype=self.dtype, device=peer.x0.device)
        h = torch.empty(rows_total, F, dtype=self.dtype, device=peer.x0.device)
        w1, b1, w2, b2, slots, n_slots = self._weights(rec)
        if peer.packed:       # rows are where the GEMMs want them; counts of my experts from the table
            rcounts = peer.allcounts[:, peer.rank * L:(peer.rank + 1) * L].contiguous().view(-1)
        else:
            rcounts = peer.counts
        desc = self._desc(M, F, W, Cs, rec, n_slots, compact=3 if peer.packed else 0)
        ws = ops.ffn_workspace(desc, peer.x0.device)
        ops.ffn_fwd_peer(desc, rcounts, peer.x0, w1, b1, w2, b2, x1, h, peer, ws, slots)
        peer.barrier()                      # every owner's output rows have landed in my ret
        if requires_grad:
            s = _Saved()
            s.x0, s.x1, s.h, s.counts, s.Cs, s.n_src = peer.x0, x1, h, rcounts, Cs, W
            s.serial = peer.serial
            self._saved = s
        return peer.ret

    def backward_peer(self, peer: PeerExchange, input_requires_grad: bool = True) -> torch.Tensor:
        """Mirror of ``forward_peer``: the combine's backward has pushed the output gradients
        into the owners' ``g`` buffers; dX's epilogue stores into the source ranks' ``dx``."""
        s = self._saved
        if s is None:
            raise RuntimeError("MOLECore.backward without a matching forward")
        if getattr(s, "serial", None) != peer.serial:
            raise RuntimeError(
                "the layer ran forward again before this backward: the push-style exchange keeps "
                "one set of buffers per layer (set MOLE_PEER_EXCHANGE=0 for such schedules)")
        W, L, Cs, M = peer.world, peer.L, peer.Cs, peer.M
        F = self._ffn_dim()
        records, _ = build_records(self.s_experts, 0, self.ebatch_size, False, 0, 0)
        rec = records[0]
        peer.barrier()                      # every rank's gradient rows have landed in my g
        dx1 = torch.empty(W * L * Cs, F, dtype=self.dtype, device=peer.g.device)
        accumulate = self._accumulate()
        w1, _, w2, _, slots, n_slots = self._weights(rec)
        desc = self._desc(M, F, W, Cs, rec, n_slots, accumulate, self.s_experts,
                          compact=3 if peer.packed else 0)
        ws = ops.ffn_workspace(desc, peer.g.device)
        grads = self.gpu_grads
        ops.ffn_bwd_peer(desc, s.counts, peer.g, s.x0, s.x1, s.h, w1, w2, dx1, peer, grads[0],
                         grads[1], grads[2], grads[3], ws, slots, slots)
        peer.barrier()                      # every owner's dX rows have landed in my dx
        ops.device_fault_poll()
        self.step += 1
        self._saved = None
        return peer.dx

    # -- helpers ---------------------------------------------------------------------------
    def _accumulate(self) -> bool:
        """GPU-resident experts' weight gradients: with ``acc_step > 1`` every backward adds to the
        gradient tensors and whoever steps the optimizer zeroes them (``acc = acc_step > 1``,
        MOLE/cpp/define.hpp:657; ``+=`` at MOLE/cpp/core.cpp:295-316); with ``acc_step == 1`` each
        backward overwrites (core.cpp:274-280)."""
        return self.acc_step > 1

    def _check_fault(self) -> None:
        """Raises if a kernel of an earlier step recorded that one of its bounded waits ran out
        (that step's activations and gradients are not to be trusted).  Reads a host copy that
        ``_poll_fault`` requested behind the previous backward: no device synchronisation."""
        if torch.cuda.is_current_stream_capturing():
            return          # no event queries while a CUDA graph is being captured (Ugraph polls behind replays)
        code = ops.device_fault_peek()
        if code:
            raise RuntimeError(
                f"a grouped-GEMM kernel gave up on a bounded wait (fault code {code}): the results "
                "of that step are invalid")

    def _desc(self, M, F, n_src, Cs, rec: Record, n_slots, accumulate=False, n_grad_slots=0,
              compact=0):
        L = self.s_experts + self.d_experts
        return ops.make_ffn_desc(self.dtype, self.act_name, self.gelu_bwd, M, F, L, n_src, Cs,
                                 rec.base_in_all, rec.base_in_all + rec.batch_size, n_slots,
                                 accumulate, self.ffn_backend, n_grad_slots, compact)

    def _weights(self, rec: Record):
        """(w1, b1, w2, b2, slot map, n_slots) for a record."""
        L = self.s_experts + self.d_experts
        slots = [0] * L
        if not rec.use_cpu_param:
            for i in range(rec.batch_size):
                slots[rec.base_in_all + i] = rec.batch_base + i
            return (*self.gpu_params, slots, self.s_experts)
        pool = _get_UniMem()
        for i in range(rec.batch_size):
            slots[rec.base_in_all + i] = rec.slots[i]
        F, M = pool.sizes[0]
        return (*pool.bases, slots, pool.pool_size)

    def _fetch_para(self, rec: Record) -> None:
        """Host-to-device fetch of a record's offloaded experts on the transfer stream
        (``_BatchRecord::fetch_para``, MOLE/cpp/core.cpp:110-143)."""
        if not rec.use_cpu_param:
            return
        pool = _get_UniMem()
        rec.ticket = pool.fetch(self.cpu_params, rec.batch_base, rec.batch_size, rec.view_base,
                                rec.prefetched)
        rec.slots = [pool.abs_slot(rec.view_base + i) for i in range(rec.batch_size)]

    # -- forward pipeline (MOLE/cpp/core.cpp:991-1131) -------------------------------------
    def can_fuse_combine(self, plan, M: int) -> bool:
        """Whether FC2's epilogue can also do the gate-weighted combine for this batch: one rank,
        bf16 on the one-CTA tensor-core kernel (fewer than 12 row tiles per expert), top-1 / top-2."""
        F = self._ffn_dim()
        return (self.world_size == 1 and self.dtype == torch.bfloat16 and self.ffn_backend in (0, 2)
                and plan.k <= 2 and plan.Cs // 128 < 12 and M % 128 == 0 and F % 128 == 0)

    def forward(self, dispatched: torch.Tensor, counts: torch.Tensor, requires_grad: bool,
                combine=None):
        """``dispatched`` ``[E_total, Cs, M]`` capacity-strided rows, ``counts`` ``[E_total]``
        valid rows per chunk -> expert outputs in the same layout.  ``combine = (plan, gates, y)``
        makes the second GEMM's epilogue add ``gates * row`` into the zeroed ``y [T, M]`` as well
        (``can_fuse_combine`` says when that is possible)."""
        self._check_fault()
        E, Cs, M = dispatched.shape
        W = self.world_size
        L = self.s_experts + self.d_experts
        assert E == L * W, "dispatched tensor does not match the expert count"
        F = self._ffn_dim()
        comp = torch.cuda.current_stream()
        multi = W > 1 or self.d_experts > 0
        sctx = ExpertStreamCtx.get(dispatched.device) if multi else None
        comm = sctx.comm_stream() if W > 1 else comp

        pool = _get_UniMem() if self.d_experts > 0 else None
        prefetched = pool.fetch_top_prefetched_batch(self.moe_id) if pool else 0
        self.fwd_base = 0
        view = pool.view_pool_size() if pool else 0
        records, groups = build_records(self.s_experts, self.d_experts, self.ebatch_size,
                                        self.use_pool, view, prefetched)
        self._records = records

        rows_total = W * L * Cs
        if W > 1:
            x0 = torch.empty(W, L, Cs, M, dtype=dispatched.dtype, device=dispatched.device)
            rcounts = torch.empty(W * L, dtype=torch.int32, device=dispatched.device)
            out_local = torch.empty_like(x0)
            ret = torch.empty_like(dispatched)
            ExpertStreamCtx.wait(comm, comp)
            with torch.cuda.stream(comm):
                MOLEDist.all2all(rcounts, counts, stream=comm)
            # No record_stream on these buffers: the compute stream joins the communication
            # stream before this method returns, so every later use or reuse of their memory on
            # the compute stream is already ordered behind the exchange.  (record_stream makes
            # the caching allocator hold the blocks back and fall through to cudaMalloc on the
            # next step: 0.2-0.9 ms per allocation.)
        else:
            x0, rcounts, out_local = dispatched, counts, torch.empty_like(dispatched)
            ret = out_local
        x1 = torch.empty(rows_total, F, dtype=dispatched.dtype, device=dispatched.device)
        h = torch.empty(rows_total, F, dtype=dispatched.dtype, device=dispatched.device)
        es = dispatched.element_size()
        chunk_bytes = Cs * M * es

        # Edges between the streams are per record, as the reference's comm_event / para_event /
        # comp_event are (MOLE/cpp/define.hpp:634-636): a record's compute waits for ITS exchange
        # and fetch, its return exchange for ITS compute, so the exchanges of later records run
        # beside the compute of earlier ones.
        for g in groups:
            arrived, computed = {}, {}
            for ri in g:
                rec = records[ri]
                if W > 1:       # first exchange of this record's experts, on the comm stream
                    MOLEDist.all2all(x0, dispatched, *exchange_geometry(rec, L, chunk_bytes), stream=comm)
                    arrived[ri] = ExpertStreamCtx.record(comm)
                self._fetch_para(rec)
            for ri in g:
                rec = records[ri]
                if W > 1:
                    ExpertStreamCtx.wait_ticket(comp, arrived[ri])
                if rec.use_cpu_param:
                    pool.wait_fetch(rec.ticket, comp)
                w1, b1, w2, b2, slots, n_slots = self._weights(rec)
                desc = self._desc(M, F, W, Cs, rec, n_slots)
                ws = ops.ffn_workspace(desc, dispatched.device)
                if combine is not None:
                    plan, gates, y = combine
                    ops.ffn_fwd_combine(desc, rcounts, x0, w1, b1, w2, b2, x1, h, out_local, plan,
                                        gates, y, ws, slots)
                else:
                    ops.ffn_fwd(desc, rcounts, x0, w1, b1, w2, b2, x1, h, out_local, ws, slots)
                if rec.use_cpu_param:
                    pool.mark_used(rec.view_base, rec.batch_size, comp)
                if W > 1:
                    computed[ri] = ExpertStreamCtx.record(comp)
            for ri in g:
                rec = records[ri]
                if W > 1:       # return exchange, on the comm stream after this record's compute
                    ExpertStreamCtx.wait_ticket(comm, computed[ri])
                    MOLEDist.all2all(ret, out_local, *exchange_geometry(rec, L, chunk_bytes), stream=comm)
        if W > 1:
            ExpertStreamCtx.wait(comp, comm)
        if requires_grad:
            s = _Saved()
            s.x0, s.x1, s.h, s.counts, s.Cs, s.n_src = x0, x1, h, rcounts, Cs, W
            self._saved = s
        return ret

    # -- backward pipeline (MOLE/cpp/core.cpp:1133-1300) -----------------------------------
    def backward(self, dout: torch.Tensor, counts: torch.Tensor, input_requires_grad: bool = True):
        s = self._saved
        if s is None:
            raise RuntimeError("MOLECore.backward without a matching forward")
        E, Cs, M = dout.shape
        W = self.world_size
        L = self.s_experts + self.d_experts
        F = self._ffn_dim()
        comp = torch.cuda.current_stream()
        multi = W > 1 or self.d_experts > 0
        sctx = ExpertStreamCtx.get(dout.device) if multi else None
        comm = sctx.comm_stream() if W > 1 else comp
        pool = _get_UniMem() if self.d_experts > 0 else None
        prefetched = pool.fetch_top_prefetched_batch(self.moe_id) if pool else 0
        self.bwd_base = 0
        view = pool.view_pool_size() if pool else 0
        records, groups = build_records(self.s_experts, self.d_experts, self.ebatch_size,
                                        self.use_pool, view, prefetched)
        es = dout.element_size()
        chunk_bytes = Cs * M * es
        rows_total = W * L * Cs
        if W > 1:
            g_local = torch.empty(W, L, Cs, M, dtype=dout.dtype, device=dout.device)
            dx_local = torch.empty_like(g_local) if input_requires_grad else None
            ret = torch.empty_like(dout) if input_requires_grad else None
            ExpertStreamCtx.wait(comm, comp)
        else:
            g_local = dout
            dx_local = torch.empty_like(dout) if input_requires_grad else None
            ret = dx_local
        dx1 = torch.empty(rows_total, F, dtype=dout.dtype, device=dout.device)
        accumulate = self._accumulate()

        instant = self.adv_adam and (self.step + 1) % self.acc_step == 0
        for g in groups:
            arrived, computed = {}, {}
            for ri in g:
                rec = records[ri]
                if W > 1:
                    MOLEDist.all2all(g_local, dout, *exchange_geometry(rec, L, chunk_bytes), stream=comm)
                    arrived[ri] = ExpertStreamCtx.record(comm)
                self._fetch_para(rec)          # weights are fetched again for backward
            for ri in g:
                rec = records[ri]
                if W > 1:
                    ExpertStreamCtx.wait_ticket(comp, arrived[ri])
                if rec.use_cpu_param:
                    pool.wait_fetch(rec.ticket, comp)
                w1, _, w2, _, slots, n_slots = self._weights(rec)
                stage = None
                if rec.use_cpu_param:
                    stage = self._take_staging(M, F, dout, comp)
                    grads, g_slots_n = stage.grads, self.ebatch_size
                    gslots = [0] * L
                    for i in range(rec.batch_size):
                        gslots[rec.base_in_all + i] = i
                    acc = False
                else:
                    grads, gslots, g_slots_n = self.gpu_grads, slots, self.s_experts
                    acc = accumulate
                desc = self._desc(M, F, W, Cs, rec, n_slots, acc, g_slots_n)
                ws = ops.ffn_workspace(desc, dout.device)
                ops.ffn_bwd(desc, s.counts, g_local, s.x0, s.x1, s.h, w1, w2, dx1, dx_local,
                            grads[0], grads[1], grads[2], grads[3], ws, slots, gslots)
                if rec.use_cpu_param:
                    pool.mark_used(rec.view_base, rec.batch_size, comp)
                    # the optimizer step of this batch right behind its backward, on the GPU
                    # (MOLE/cpp/core.cpp:1216-1227), or the gradients back to the host
                    n_adam = min(rec.batch_size, self.hybrid_adam_count - rec.batch_base) if instant else 0
                    if n_adam > 0:
                        self._instant_adam(rec, n_adam, stage, comp)
                    if n_adam < rec.batch_size:
                        self._store_grad(rec, grads, comp, first=max(n_adam, 0))
                    stage.release(sctx.tran_back_stream())
                if W > 1:
                    computed[ri] = ExpertStreamCtx.record(comp)
            for ri in g:
                rec = records[ri]
                if W > 1 and input_requires_grad:
                    ExpertStreamCtx.wait_ticket(comm, computed[ri])
                    MOLEDist.all2all(ret, dx_local, *exchange_geometry(rec, L, chunk_bytes), stream=comm)
        if W > 1:
            ExpertStreamCtx.wait(comp, comm)
        if self.d_experts > 0:
            check(lib.mole_ctx_synchronize(sctx.handle, 4))     # D2H stores done
            self._finish_grad_accumulate()
        ops.device_fault_poll()
        self.step += 1
        self.unset_lazy_zero()
        self._saved = None
        return ret

    # -- offloaded-expert gradients (MOLE/cpp/core.cpp:77-103, uparameter.cpp:68-83) ---------
    def _take_staging(self, M, F, like, comp) -> "_Staging":
        """Device block that receives one record's weight gradients (and, for the GPU optimizer
        step, its Adam moments).  Two blocks alternate, each guarded by an event: the compute of
        record i+1 writes the other block while record i's block is still travelling to the host,
        and waits only for the device-to-host copies of record i-1."""
        if not self._staging:
            self._staging = [_Staging(self.ebatch_size, M, F, like.dtype, like.device) for _ in range(2)]
        st = self._staging[self._staging_turn]
        self._staging_turn ^= 1
        st.acquire(comp)
        return st

    def _store_grad(self, rec: Record, grads, comp, first: int = 0) -> None:
        """Gradients of the record's experts ``[first, batch_size)`` to the pinned host arrays on
        the device-to-host stream (``store_grad``, MOLE/cpp/core.cpp:77-103)."""
        sctx = ExpertStreamCtx.get(grads[0].device)
        lazy = getattr(self.cpu_grads[0], "lazy_zero", True)
        for p_id in range(4):
            host = self.cpu_grads[p_id][rec.batch_base + first:rec.batch_base + rec.batch_size]
            dev = grads[p_id][first:rec.batch_size]
            nbytes = host.numel() * host.element_size()
            if self.acc_step > 1 and not lazy:
                stage = torch.empty_like(host).pin_memory()
                check(lib.mole_store_to_host(sctx.handle, C.c_void_p(stage.data_ptr()),
                                             C.c_void_p(dev.data_ptr()), nbytes,
                                             C.c_void_p(comp.cuda_stream)))
                self._pending_acc.append((host, stage))
            else:
                check(lib.mole_store_to_host(sctx.handle, C.c_void_p(host.data_ptr()),
                                             C.c_void_p(dev.data_ptr()), nbytes,
                                             C.c_void_p(comp.cuda_stream)))

    def _instant_adam(self, rec: Record, n: int, stage: "_Staging", comp) -> None:
        """Adam step of the record's first ``n`` experts on the GPU, right behind their backward
        (``_MOLECore::instant_adam``, MOLE/cpp/core.cpp:848-943): the moments come in on the
        host-to-device stream behind the compute, one fused kernel per parameter kind updates the
        weights where they lie in the pool slots, and parameters and moments go back to the
        pinned host arrays on the device-to-host stream.  With ``acc_step > 1`` the gradient the
        host has accumulated over the earlier micro-steps is brought in and added
        (core.cpp:906-918)."""
        pool = _get_UniMem()
        sctx = ExpertStreamCtx.get(stage.grads[0].device)
        tran, back = sctx.tran_stream(), sctx.tran_back_stream()
        a = self.adam
        base = rec.batch_base
        lazy = getattr(self.cpu_grads[0], "lazy_zero", True)
        extra = self.acc_step > 1 and not lazy
        stage.ensure_moments(extra)
        ExpertStreamCtx.wait(tran, comp)            # gradients written, weights no longer read
        a0 = rec.slots[0]
        with torch.cuda.stream(tran):
            for k in range(4):
                stage.m[k][:n].copy_(self.cpu_mome[k][base:base + n], non_blocking=True)
                stage.v[k][:n].copy_(self.cpu_vari[k][base:base + n], non_blocking=True)
                if extra:
                    stage.g_host[k][:n].copy_(self.cpu_grads[k][base:base + n], non_blocking=True)
            for k in range(4):
                per = stage.grads[k][0].numel()
                es = stage.grads[k].element_size()
                p_ptr = pool.bases[k] + a0 * per * es
                check(lib.mole_adam_update(
                    C.c_void_p(p_ptr), C.c_void_p(stage.m[k].data_ptr()),
                    C.c_void_p(stage.v[k].data_ptr()), C.c_void_p(stage.grads[k].data_ptr()),
                    C.c_void_p(stage.g_host[k].data_ptr()) if extra else None, n * per,
                    ops._DTYPES[self.dtype], a["beta1"], a["beta2"], a["t"] + 1, a["lr"], a["lam"],
                    a["eps"], int(a["adamW"]), C.c_void_p(tran.cuda_stream)))
        for k in range(4):
            per = stage.grads[k][0].numel()
            es = stage.grads[k].element_size()
            nbytes = n * per * es
            for host, dev_ptr in ((self.cpu_params[k], pool.bases[k] + a0 * per * es),
                                  (self.cpu_mome[k], stage.m[k].data_ptr()),
                                  (self.cpu_vari[k], stage.v[k].data_ptr())):
                check(lib.mole_store_to_host(sctx.handle, C.c_void_p(host[base:base + n].data_ptr()),
                                             C.c_void_p(dev_ptr), nbytes,
                                             C.c_void_p(tran.cuda_stream)))
        # a later fetch into these slots waits until the updated weights have left them
        pool.mark_used(rec.view_base, rec.batch_size, back)
        # the next host-to-device copy into this block's moments must not overtake these stores
        ExpertStreamCtx.wait(tran, back)

    def _finish_grad_accumulate(self) -> None:
        for host, stage in self._pending_acc:
            host += stage
        self._pending_acc = []

    def _ffn_dim(self) -> int:
        for t in (self.gpu_params[0], self.cpu_params[0]):
            if t is not None and not isinstance(t, int):
                return t.shape[1]
        raise RuntimeError("no expert parameters registered")
