"""N-sharded multi-GPU use of the path (one process per GPU).

The GEMM shards along N: rank r owns output columns [r*N/P, (r+1)*N/P), i.e. rows of the
quantised weight.  K is never split, so every output element is computed exactly as on one
GPU.  What has to travel is the quantised activation; outputs stay sharded unless the caller
gathers them.  The transfers are made by the C ABI (include/mixedgemm_c.h, csrc/dist.cu):

  Communicator   NCCL collectives through mg_dist_* / mg_bcast_activations / mg_allgather_*:
                 "quantise once, broadcast", or "quantise M/P rows each, all-gather"
  PushExchange   the overlapped exchange: every rank quantises M/P rows in place in its own block
                 of a buffer that is laid out rank by rank, and pushes the block into every
                 peer's buffer over NVLink - one copy-engine copy per peer (mg_push_shard) or one
                 kernel with plain peer stores (mg_push_block); the GEMM waits, row shard by row
                 shard, for the flags that follow the data

The only thing the host framework (torch.distributed) is used for is handing small byte strings
from rank to rank at set-up time: the NCCL id and the IPC handles of the exchange buffers.
The shard bookkeeping (shard_range, sf_shard, shard_weights, activation_shard) is plain tensor
slicing and works on CPU tensors too.  The reference has no multi-GPU mode.  The GEMM and the
quantiser never have another GPU's memory as an operand; only the push kernel stores into it.
"""
import ctypes

import torch

from . import _capi


# ----------------------------------------------------------------------------- shard bookkeeping
def shard_range(N, world, rank):
    """(first row, row count) of `rank`'s weight shard.  Shards are whole 128-row scale blocks."""
    if N % (128 * world) != 0:
        raise ValueError("N = %d cannot be split into %d shards of whole 128-row blocks" % (N, world))
    n = N // world
    return rank * n, n


def sf_shard(sf, N, kseg, world, rank):
    """The slice of a swizzled weight-scale buffer that belongs to `rank`'s rows: scale atoms of a
    128-row block are contiguous, so a row shard is a contiguous byte range."""
    r0, n = shard_range(N, world, rank)
    per_block = ((kseg + 127) // 128) * 512
    return sf[(r0 // 128) * per_block:((r0 + n) // 128) * per_block]


def shard_weights(B, N, KN, KS, KO, world, rank):
    """B = (BN, BS, BO, SFBN, SFBS, SFBO) of the full weight -> the same six for `rank`'s shard
    (views, no copy)."""
    r0, n = shard_range(N, world, rank)
    return (B[0][r0:r0 + n], B[1][r0:r0 + n], B[2][r0:r0 + n],
            sf_shard(B[3], N, KN, world, rank), sf_shard(B[4], N, KS, world, rank), sf_shard(B[5], N, KO, world, rank))


def _pitched_base(t):
    """[rows, pitch] buffer under a [rows, logical] row-pitched view (or the tensor itself)."""
    if t.is_contiguous():
        return t
    return t.as_strided((t.size(0), t.stride(0)), (t.stride(0), 1), t.storage_offset())


def activation_shard(A, M, split, world, rank):
    """Views of the six full-size activation buffers that hold rows [rank*M/P, (rank+1)*M/P):
    what this rank's quantiser writes when the quantisation itself is sharded along M.  M/P must
    be a multiple of 128 so that a shard is whole scale blocks."""
    if M % (128 * world) != 0:
        raise ValueError("M = %d cannot be split into %d shards of whole 128-row blocks" % (M, world))
    mp = M // world
    r0 = rank * mp
    out = [A[i][r0:r0 + mp] for i in range(3)]
    for i, k in enumerate(split):
        per_block = ((k + 127) // 128) * 512
        out.append(A[3 + i][(r0 // 128) * per_block:((r0 + mp) // 128) * per_block])
    return tuple(out)


def shard_byte_ranges(A, M, split, world, rank):
    """[(tensor, first byte, byte count), ...]: where rank's M/P rows live inside each of the six
    buffers of a quantised activation (codes: rows x pitch; scales: whole 128-row blocks)."""
    mp = M // world
    out = []
    for i in range(3):
        base = _pitched_base(A[i])
        pitch = base.stride(0) if base.numel() else 0
        out.append((base, rank * mp * pitch, mp * pitch))
    for i, k in enumerate(split):
        per_block = ((k + 127) // 128) * 512
        out.append((A[3 + i], (rank * mp // 128) * per_block, (mp // 128) * per_block))
    return out


def _vp_array(values):
    return (ctypes.c_void_p * len(values))(*values)


def _sz_array(values):
    return (ctypes.c_size_t * len(values))(*values)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _exchange_bytes(payload, group=None):
    """Every rank contributes a byte string; returns the list of all of them (set-up time only)."""
    import torch.distributed as dist
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, payload, group=group)
    return out


# ----------------------------------------------------------------------------- NCCL through the C ABI
class Communicator:
    """An NCCL communicator owned by the library (mg_dist_init).  The 128-byte id is made on rank 0
    and handed to the others through `group` (a torch.distributed group over any backend)."""

    def __init__(self, world, rank, group=None):
        import torch.distributed as dist
        self.lib = _capi.load()
        self.world, self.rank = world, rank
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            _capi.check(self.lib.mg_dist_unique_id(ident), "mg_dist_unique_id")
        box = [ident.raw]
        dist.broadcast_object_list(box, src=0, group=group)
        self.handle = ctypes.c_void_p()
        _capi.check(self.lib.mg_dist_init(ctypes.byref(self.handle), box[0], world, rank), "mg_dist_init")

    def close(self):
        if self.handle:
            self.lib.mg_dist_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def broadcast_activations(self, A, src=0):
        """The six quantised-activation buffers go from `src` into every rank's own memory in one
        grouped broadcast (row-pitched views are sent with their padding)."""
        bufs = [_pitched_base(t) for t in A if t.numel()]
        _capi.check(self.lib.mg_bcast_activations(
            self.handle, src, _vp_array([t.data_ptr() for t in bufs]),
            _sz_array([t.numel() * t.element_size() for t in bufs]), len(bufs), _stream()), "mg_bcast_activations")

    def all_gather_activations(self, A, M, split):
        """Every rank has quantised its own M/P rows in place (activation_shard); gather the others'."""
        ptrs, shard = [], []
        for t, first, count in shard_byte_ranges(A, M, split, self.world, 0):
            if count:
                ptrs.append(t.data_ptr())
                shard.append(count)
        _capi.check(self.lib.mg_allgather_inplace(self.handle, _vp_array(ptrs), _sz_array(shard), len(ptrs), _stream()),
                    "mg_allgather_inplace")

    def all_gather_output(self, Y_local):
        """[M, N/P] shards -> [M, N] (only for callers that need the whole output)."""
        Yl = Y_local.contiguous()
        parts = torch.empty((self.world,) + tuple(Yl.shape), dtype=Yl.dtype, device=Yl.device)
        _capi.check(self.lib.mg_allgather_output(self.handle, Yl.data_ptr(), parts.data_ptr(),
                                                 Yl.numel() * Yl.element_size(), _stream()), "mg_allgather_output")
        return torch.cat(list(parts), dim=1)


# ----------------------------------------------------------------------------- the overlapped exchange
class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def _align(n, a=1024):
    return (n + a - 1) // a * a


def exchange_layout(shapes, world):
    """Where things lie in one buffer set of the overlapped exchange (host arithmetic only).
    shapes = [(M, (KN, KS, KO)), ...], the activations of a step.  Returns (parts, block_bytes,
    flag_off, total_bytes): the set is `world` blocks of block_bytes (block r = what rank r quantises)
    followed by `world` int32 flags at flag_off; parts[i] = (rows per rank, logical row bytes of the
    three code tensors, their row pitches, byte sizes of the six parts, their offsets inside a block)
    for activation i.  Every part starts on a 1 KB boundary, which the tensor maps (32 bytes), the
    scale copies (16) and the 16-byte loads of the push kernel all accept."""
    lib = _capi.load()
    parts, off = [], 0
    for (M, split) in shapes:
        if M % (256 * world) != 0:
            raise ValueError("M = %d must split into %d shards of whole 256-row blocks" % (M, world))
        mp = M // world
        logical = (split[0] // 2, split[1] // 4 * 3, split[2])
        pitch = [lib.mg_code_pitch(0, i, k) for i, k in enumerate(split)]
        sizes = [mp * p for p in pitch] + [lib.mg_sf_bytes(mp, k) for k in split]
        offs = []
        for n in sizes:
            offs.append(off)
            off += _align(n)
        parts.append((mp, logical, pitch, sizes, offs))
    flag_off = world * off
    return parts, off, flag_off, flag_off + _align(4 * world)


class PushExchange:
    """Exchange buffers for `n_sets` steps' worth of quantised activations (shapes = [(M, (KN, KS, KO)), ...],
    the activations of one step).  A set is one device allocation, laid out identically on every rank
    and opened on every other rank through CUDA IPC.  It is stored rank by rank: everything rank r
    quantises in a step - its M/P rows of every activation, each as three code tensors at their row
    pitch followed by their three scale tensors - is ONE contiguous block, followed by `world` flag
    words.  A step's push is then either one kernel that reads the block once and stores it into every
    peer's set (mode "sm", mg_push_block, on `push_ctas` SMs that it keeps to itself: launch the GEMM
    that runs beside it with option GEMM_MAX_CLUSTERS = SM pairs - push_ctas / 2; push_ctas = 0 uses
    every SM and is for a push that runs alone), or one large copy-engine copy per peer (mode
    "ce", mg_push_shard: small copies reach a fraction of the NVLink rate, every copy costs tens of
    microseconds of latency, and copies to several peers at once share the engines badly).  The GEMM
    reads that layout in place (api.ShardedActivation).

    How many sets: a rank may run ahead of a peer by the steps the caller keeps in flight.  When a
    step pushes, multiplies and joins the same set, 2 sets are enough; when the push of step i + 1 is
    issued before the GEMM of step i (so that the transfer hides under it), a set is overwritten three
    steps after it was read and 4 are needed."""

    def __init__(self, shapes, world, rank, device, n_sets=2, group=None, mode="sm", push_ctas=8, ce_peers=2):
        from .api import ShardedActivation
        if mode not in ("sm", "ce", "hybrid"):
            raise ValueError("mode is 'sm' (a kernel stores into the peers' buffers), 'ce' (copy engines) or "
                             "'hybrid' (copy engines for the `ce_peers` farthest peers, the kernel for the rest)")
        self.ce_peers = min(ce_peers, max(world - 2, 0)) if mode == "hybrid" else 0
        self.lib = lib = _capi.load()
        self.world, self.rank, self.device = world, rank, device
        self.mode, self.push_ctas = mode, push_ctas
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.shapes = list(shapes)
        self.epoch = torch.zeros(n_sets, dtype=torch.int32, device=device)
        self.streams = [torch.cuda.Stream(device=device) for _ in range(max(world - 1, 1))]
        self.sets = []
        handles = []
        parts, off, self.flag_off, total = exchange_layout(self.shapes, world)
        self.block_bytes = off
        with torch.cuda.device(device):
            for s in range(n_sets):
                ptr = ctypes.c_void_p()
                _capi.check(lib.mg_xbuf_alloc(ctypes.byref(ptr), total), "mg_xbuf_alloc")
                h = ctypes.create_string_buffer(64)
                _capi.check(lib.mg_ipc_export(ptr, h), "mg_ipc_export")
                handles.append(h.raw)
                flat = torch.as_tensor(_Raw(ptr.value, total), device=device)
                acts = []
                for (mp, logical, pitch, sizes, offs) in parts:
                    shards = []
                    for r in range(world):
                        blk = flat[r * off:(r + 1) * off]
                        A = []
                        for i in range(3):
                            v = blk[offs[i]:offs[i] + sizes[i]].view(mp, pitch[i])
                            A.append(v[:, :logical[i]] if pitch[i] != logical[i] else v)
                        for i in range(3):
                            A.append(blk[offs[3 + i]:offs[3 + i] + sizes[3 + i]])
                        shards.append(tuple(A))
                    acts.append(ShardedActivation(shards))
                flags = flat[self.flag_off:self.flag_off + 4 * world].view(torch.int32)
                self.sets.append(dict(ptr=ptr, A=acts, flags=flags, bases=None, flat=flat))
        # every rank opens every other rank's sets
        self._imported = []
        all_handles = _exchange_bytes(handles, group) if world > 1 else [handles]
        for k, b in enumerate(self.sets):
            bases = []
            for r in range(world):
                if r == rank:
                    bases.append(b["ptr"].value)
                else:
                    p = ctypes.c_void_p()
                    with torch.cuda.device(device):
                        _capi.check(lib.mg_ipc_import(all_handles[r][k], ctypes.byref(p)), "mg_ipc_import")
                    self._imported.append(p)
                    bases.append(p.value)
            b["bases"] = bases

    def buffers(self, set_index, i):
        """Activation i of set `set_index` as the api.ShardedActivation that matmul_multi takes."""
        return self.sets[set_index]["A"][i]

    def shard(self, set_index, i, rank=None):
        """The six tensors of this rank's (or `rank`'s) M/P rows of activation i: what its quantiser
        writes (`out=` of reorder_quantize_x)."""
        return self.sets[set_index]["A"][i].shards[self.rank if rank is None else rank]

    def begin_step(self, set_index):
        """Before the quantisers that fill set `set_index`: the value its flags will carry this time."""
        _capi.check(self.lib.mg_epoch_bump(self.epoch[set_index:].data_ptr(), _stream()), "mg_epoch_bump")

    def push(self, set_index):
        """After this rank's rows of every activation of the set have been quantised on the current
        stream: copy its block into every peer's set and raise this rank's flag there.  The copies run
        on the exchange's own streams, ordered after the current stream's work so far."""
        b = self.sets[set_index]
        done = torch.cuda.Event()
        done.record()
        if self.mode in ("sm", "hybrid"):
            # one kernel on one side stream; in the hybrid form the copy engines take the peers farthest
            # down the ring (one stream each) and the kernel the others
            nring = self.world - 1
            ce_steps = list(range(nring - self.ce_peers + 1, nring + 1))
            sm_mask = 0
            if ce_steps:
                for step in range(1, nring - self.ce_peers + 1):
                    sm_mask |= 1 << (step - 1)
            st = self.streams[0]
            st.wait_event(done)
            _capi.check(self.lib.mg_push_block_to(
                self.world, self.rank, sm_mask, _vp_array(b["bases"]), self.rank * self.block_bytes, self.block_bytes,
                self.flag_off, self.epoch[set_index:].data_ptr(), self.counter.data_ptr(), self.push_ctas,
                st.cuda_stream), "mg_push_block")
            for j, step in enumerate(ce_steps):
                cs = self.streams[1 + j]
                cs.wait_event(done)
                per_step = [cs.cuda_stream] * nring
                _capi.check(self.lib.mg_push_shard_to(
                    self.world, self.rank, 1 << (step - 1), _vp_array(b["bases"]), _sz_array([self.rank * self.block_bytes]),
                    _sz_array([self.block_bytes]), 1, self.flag_off, self.epoch[set_index:].data_ptr(),
                    _vp_array(per_step)), "mg_push_shard")
            return
        for st in self.streams:
            st.wait_event(done)
        _capi.check(self.lib.mg_push_shard(
            self.world, self.rank, _vp_array(b["bases"]), _sz_array([self.rank * self.block_bytes]),
            _sz_array([self.block_bytes]), 1, self.flag_off, self.epoch[set_index:].data_ptr(),
            _vp_array([st.cuda_stream for st in self.streams])), "mg_push_shard")

    def ready(self, set_index, i):
        """The `flags` entry of api.matmul_multi for a problem that reads activation i of the set: one
        flag per rank, target = the set's current epoch, tiles start with this rank's own rows."""
        b = self.sets[set_index]
        mp = b["A"][i].shard_rows
        return (b["flags"], self.epoch[set_index:set_index + 1], mp, self.rank * mp)

    def join(self):
        """Make the current stream wait for the copies this rank has issued (the buffers it pushed
        FROM may be overwritten afterwards)."""
        for st in self.used_streams():
            torch.cuda.current_stream().wait_stream(st)

    def used_streams(self):
        """The side streams a push puts work on."""
        if self.mode == "ce":
            return self.streams
        return self.streams[:1 + self.ce_peers]

    def close(self):
        torch.cuda.synchronize(self.device)
        for p in self._imported:
            self.lib.mg_ipc_close(p)
        self._imported = []
        for b in self.sets:
            b["A"] = b["flags"] = b["flat"] = None
            self.lib.mg_xbuf_free(b["ptr"])
        self.sets = []
