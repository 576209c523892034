"""Expert-parallel communicator (interface of MOLE/utils/Udist.py:6-64).

``MOLEDist(local_rank=...)`` is a singleton.  When ``torch.distributed`` is initialised it
creates the library's own NCCL communicator: rank 0 makes the 128-byte unique id, the bytes
travel through ``torch.distributed`` (any backend) and every rank calls ``mole_comm_create``
-- the reference reached the same point by casting the c10d process group
(MOLE/cpp/communication.cpp:19-66).  ``all2all`` is the equal-split grouped send/recv of
MOLE/cpp/communication.cpp:68-100 on raw bytes.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .._lib import check, lib


class MOLEDist:
    _instance = None

    def __new__(cls, *args, **kw):
        if cls._instance is None:
            inst = object.__new__(cls)
            inst.comm = None
            if dist.is_initialized():
                inst.world_size = dist.get_world_size()
                inst.use_distributed = inst.world_size > 1
                inst.rank = dist.get_rank()
                inst.local_rank = kw["local_rank"]
                inst.device = torch.device("cuda", inst.local_rank)
                ranks = kw.get("MOLE_group_ranks", list(range(inst.world_size)))
                inst.MOLE_group = dist.new_group(ranks=ranks)
                if inst.use_distributed:
                    inst.comm = cls._make_comm(inst)
            else:
                inst.world_size = 1
                inst.use_distributed = False
                inst.rank = 0
                inst.local_rank = kw.get("local_rank", 0)
                inst.device = torch.device("cuda", inst.local_rank)
                inst.MOLE_group = None
            cls._instance = inst
        return cls._instance

    @staticmethod
    def _make_comm(inst):
        ident = (C.c_uint8 * 128)()
        if inst.rank == 0:
            check(lib.mole_comm_unique_id(ident))
        # the id travels as a CPU or CUDA tensor depending on the process group's backend
        backend = dist.get_backend(inst.MOLE_group)
        dev = inst.device if backend == "nccl" else torch.device("cpu")
        t = torch.tensor(list(ident), dtype=torch.uint8, device=dev)
        dist.broadcast(t, src=0, group=inst.MOLE_group)
        ident = (C.c_uint8 * 128)(*t.cpu().tolist())
        handle = C.c_void_p()
        check(lib.mole_comm_create(ident, inst.world_size, inst.rank, inst.local_rank,
                                   C.byref(handle)))
        return handle

    @staticmethod
    def enabled():
        return MOLEDist._instance.use_distributed

    @staticmethod
    def all2all(recv: torch.Tensor, send: torch.Tensor, bytes_per_peer: int = -1,
                peer_stride_bytes: int = -1, byte_offset: int = 0, stream=None) -> None:
        """Chunk q of ``send`` goes to rank q; chunk r of ``recv`` comes from rank r."""
        inst = MOLEDist._instance
        total = send.numel() * send.element_size()
        if peer_stride_bytes < 0:
            peer_stride_bytes = total // inst.world_size
        if bytes_per_peer < 0:
            bytes_per_peer = peer_stride_bytes
        st = (stream or torch.cuda.current_stream()).cuda_stream
        if inst.comm is None:
            if inst.world_size != 1:
                raise RuntimeError("MOLEDist has no communicator")
            recv.view(torch.uint8).view(-1)[byte_offset:byte_offset + bytes_per_peer].copy_(
                send.view(torch.uint8).view(-1)[byte_offset:byte_offset + bytes_per_peer],
                non_blocking=True)
            return
        check(lib.mole_all2all(inst.comm, C.c_void_p(send.data_ptr() + byte_offset),
                               C.c_void_p(recv.data_ptr() + byte_offset), bytes_per_peer,
                               peer_stride_bytes, C.c_void_p(st)))

    @staticmethod
    def all2allsingle(rec_lst, inp_lst):
        dist.all_to_all_single(rec_lst, inp_lst, group=MOLEDist._instance.MOLE_group)

    @staticmethod
    def get_MOLE_world_size():
        return MOLEDist._instance.world_size

    @staticmethod
    def get_MOLE_local_rank():
        return MOLEDist._instance.local_rank

    @staticmethod
    def get_MOLE_rank():
        return MOLEDist._instance.rank

    @staticmethod
    def get_MOLE_device():
        return MOLEDist._instance.device
