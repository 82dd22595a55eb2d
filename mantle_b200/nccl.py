"""A communicator for mantleCudaSampleVocabSharded (include/mantle_cuda_sampler_nccl.h), made
with NCCL's own calls through ctypes: ncclGetUniqueId on one rank, the id handed to the others
by whatever channel the host already has (here: torch.distributed's object broadcast), then
ncclCommInitRank on every rank.  A Go host does the same three steps over its own channel.

The reference has no counterpart (it links no collective library,
internal/backend/cuda/native/runtime.go:6).
"""
import ctypes as C

from . import build as _build

_nccl = None
_lib = None


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]  # ncclUniqueId, nccl.h: NCCL_UNIQUE_ID_BYTES


def _libnccl():
    """libnccl by its soname: the copy torch already mapped when there is one, else the system's."""
    global _nccl
    if _nccl is None:
        L = C.CDLL("libnccl.so.2")
        L.ncclGetUniqueId.restype = C.c_int
        L.ncclGetUniqueId.argtypes = [C.POINTER(UniqueId)]
        L.ncclCommInitRank.restype = C.c_int
        L.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        L.ncclCommDestroy.restype = C.c_int
        L.ncclCommDestroy.argtypes = [C.c_void_p]
        L.ncclGetErrorString.restype = C.c_char_p
        L.ncclGetErrorString.argtypes = [C.c_int]
        _nccl = L
    return _nccl


def _check(code, where):
    if code != 0:
        raise RuntimeError("%s failed: ncclResult %d (%s)" % (where, code, _libnccl().ncclGetErrorString(code).decode()))


def load():
    """Loads libmantle_cuda_sampler_nccl.so (building it first when nvcc is at hand and it is stale)."""
    global _lib
    if _lib is not None:
        return _lib
    import os

    from . import native

    native.load()
    _libnccl()
    try:
        _build.build_nccl()
    except Exception:
        if not os.path.exists(_build.NCCL_LIB_PATH):
            raise
    L = C.CDLL(_build.NCCL_LIB_PATH)
    f = L.mantleCudaSampleVocabSharded
    f.restype = C.c_int
    f.argtypes = [C.POINTER(native.SampleBatch), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                  C.POINTER(C.c_int)]
    _lib = L
    return L


def new_unique_id():
    uid = UniqueId()
    _check(_libnccl().ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
    return C.string_at(C.byref(uid), 128)  # all 128 bytes: the id is binary, not a C string


class Communicator:
    """ncclComm_t of this rank.  The current CUDA device must be the rank's GPU."""

    def __init__(self, world_size, rank, unique_id_bytes):
        uid = UniqueId()
        C.memmove(C.byref(uid), unique_id_bytes, 128)
        self.handle = C.c_void_p()
        _check(_libnccl().ncclCommInitRank(C.byref(self.handle), world_size, uid, rank), "ncclCommInitRank")
        self.world_size, self.rank = world_size, rank

    def close(self):
        if self.handle:
            _libnccl().ncclCommDestroy(self.handle)
            self.handle = C.c_void_p()


def communicator_from_torch(group=None):
    """A communicator over the ranks of a torch.distributed group: rank 0 makes the id, the
    group's own object broadcast carries it."""
    import torch.distributed as dist

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [new_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return Communicator(world, rank, box[0])
