"""Column-parallel W4A4 linear: the output channels (weight rows) of one layer are split into
contiguous blocks over the ranks of a torch.distributed group, one process per GPU.

The reference has no multi-GPU code. The layer shards naturally: output column n depends only on
weight row n, its per-channel vectors and the (replicated) activations. Every rank quantizes the
activations itself, so codes and per-token scales are bit-identical everywhere, computes its
[M, N/G] block with the fused kernel, and the blocks are exchanged with ONE all-gather (NCCL on
GPUs, gloo in the CPU tests of the host logic). Results equal the unsharded layer bit for bit;
the dual-uniform selectors, which depend on the GLOBAL output column, receive the shard's
column offset.
"""
import ctypes
import os

import torch
import torch.distributed as dist


def shard_bounds(n_out: int, world: int, rank: int):
    """[begin, end) of the output channels owned by `rank`. Blocks are contiguous and as even as
    possible, each a multiple of 8 channels wide (16-byte fp16 row segments) except possibly the
    last."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    per = -(-n_out // world)
    per = -(-per // 8) * 8
    b = min(n_out, rank * per)
    return b, min(n_out, b + per)


def shard_rows(t: torch.Tensor, world: int, rank: int):
    """Rows [begin,end) of a per-channel tensor ([N, ...]) for `rank`."""
    b, e = shard_bounds(t.shape[0], world, rank)
    return t[b:e].contiguous()


def gather_columns(local: torch.Tensor, n_out: int, group=None, out: torch.Tensor = None):
    """All-gather of the column blocks: `local` is this rank's [M, n_local] block (n_local per
    shard_bounds); returns the row-major [M, n_out] tensor on every rank. Even shards take one
    all_gather_into_tensor plus one strided copy; ragged shards (last rank narrower) are padded to
    the common width first."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    M = local.shape[0]
    width = shard_bounds(n_out, world, 0)[1]
    b, e = shard_bounds(n_out, world, rank)
    if local.shape[1] != e - b:
        raise ValueError(f"rank {rank}: block has {local.shape[1]} columns, shard_bounds says {e - b}")
    if e - b != width:
        padded = local.new_zeros((M, width))
        padded[:, : e - b] = local
        local = padded
    gathered = local.new_empty((world, M, width))
    dist.all_gather_into_tensor(gathered.view(world * M, width), local.contiguous(), group=group)
    full = gathered.permute(1, 0, 2).reshape(M, world * width)
    if world * width != n_out:
        full = full[:, :n_out]
    if out is not None:
        out.copy_(full)
        return out
    return full.contiguous()


class SharedHostTensor:
    """One HOST tensor that every rank process of a node maps: POSIX shared memory (a file under
    /dev/shm) mapped MAP_SHARED, and -- with pin=True -- page-locked for the calling process's GPU
    (cudaHostRegister), so that each rank's copy engine moves its own slice of the job over its own PCIe
    link. The job of an N-sharded layer whose activations and result live on the host has ONE input and ONE
    result: every rank reads the same activations from this memory and delivers its [M, N/G] column block
    straight into columns [r*N/G, (r+1)*N/G) of the one row-major [M, N] result (`host_result_slice`); no
    device-side gather and no second host copy are involved.

    Exactly one process passes create=True (and calls it first; the others open after a barrier). `close()`
    unpins and unmaps; the creator also removes the file."""

    def __init__(self, name, shape, dtype, create, pin=True):
        self.path = os.path.join("/dev/shm", name)
        self.create, self.pinned = create, False
        numel = 1
        for d in shape:
            numel *= int(d)
        if create and os.path.exists(self.path):
            os.unlink(self.path)
        if not create and not os.path.exists(self.path):
            raise FileNotFoundError(f"{self.path}: the creating rank has not made it yet (barrier missing?)")
        self.tensor = torch.from_file(self.path, shared=True, size=numel, dtype=dtype).view(*shape)
        self.nbytes = numel * self.tensor.element_size()
        if pin:
            rc = torch.cuda.cudart().cudaHostRegister(self.tensor.data_ptr(), self.nbytes, 0)
            if int(rc) != 0:
                raise RuntimeError(f"cudaHostRegister({self.path}) failed with CUDA error {int(rc)}")
            self.pinned = True

    def close(self):
        if self.pinned:
            torch.cuda.cudart().cudaHostUnregister(self.tensor.data_ptr())
            self.pinned = False
        self.tensor = None
        if self.create and os.path.exists(self.path):
            os.unlink(self.path)


def host_result_slice(n_out: int, world: int, rank: int):
    """Where rank `rank` delivers its block inside the one row-major fp16 [M, n_out] host result:
    (byte offset of its first column from the start of a row, row pitch in elements, block width)."""
    b, e = shard_bounds(n_out, world, rank)
    return 2 * b, n_out, e - b


class PeerOutput:
    """A [M, N] fp16 result buffer that exists on every rank and is mapped into every other
    rank's address space (torch symmetric memory over NVLink). The GEMM epilogue of each rank
    stores its column block straight into all of these buffers (`duq4_epilogue.out_peers`), so
    the all-gather is fused into the kernel: no separate collective, no re-layout copy. Where the
    NVLink switch offers a multicast mapping of the buffer (NVLS), the epilogue stores each 16-byte
    row segment ONCE to that mapping (`duq4_epilogue.out_multicast`, multimem.st) and the switch
    replicates it, which cuts a rank's NVLink egress from (G-1)/G of the result to 1/G of it.

    `barrier()` is the library's own device-side barrier across the ranks on the current stream
    (duq4_peer_barrier): flags in symmetric memory, a bounded wait (`barrier_timeout_ns`, 0 = one
    second) and a status word instead of a hang when a rank does not arrive."""

    def __init__(self, M, N, device, group=None, use_multicast=True, barrier_timeout_ns=0):
        import torch.distributed._symmetric_memory as symm
        from . import lib as L
        self._L = L
        self.M, self.N = M, N
        grp = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(grp), dist.get_rank(grp)
        if self.world > 8:
            raise ValueError("fused all-gather supports at most 8 ranks")
        self.buf = symm.empty((M, N), dtype=torch.float16, device=device)
        self.hdl = symm.rendezvous(self.buf, grp)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc if use_multicast else 0
        # barrier flags: world uint64 slots per rank, slot s of rank r is written by rank s
        self.flags = symm.empty((self.world,), dtype=torch.int64, device=device)
        self.flags.zero_()
        self.fhdl = symm.rendezvous(self.flags, grp)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self.fhdl.buffer_ptrs])
        self.epoch = 0
        self.barrier_timeout_ns = int(barrier_timeout_ns)
        torch.cuda.synchronize(device)
        dist.barrier(grp)   # every rank's flags are zero before anybody's first flag store can land

    def column_ptrs(self, col_begin):
        return [p + 2 * col_begin for p in self.ptrs]

    def multicast_column_ptr(self, col_begin):
        return self.multicast_ptr + 2 * col_begin if self.multicast_ptr else 0

    def barrier(self, arrive=True):
        """Queues the barrier on the current stream. arrive=False only advances the epoch without
        launching (a rank that stays away -- used to exercise the time-out path of the others)."""
        self.epoch += 1
        if not arrive:
            return
        with torch.cuda.device(self.buf.device):
            self._L.call("duq4_peer_barrier", self._flag_ptrs, self.world, self.rank, self.epoch, self.barrier_timeout_ns,
                         self._L.current_stream())

    def catch_up(self):
        """After a barrier this rank stayed away from: publish the current epoch so that the peers' later
        barriers see this rank as arrived (a barrier launch whose own wait is already satisfied or bounded)."""
        with torch.cuda.device(self.buf.device):
            self._L.call("duq4_peer_barrier", self._flag_ptrs, self.world, self.rank, self.epoch, self.barrier_timeout_ns,
                         self._L.current_stream())


class ColumnParallelLinear4bit(torch.nn.Module):
    """One W4A4 layer sharded over a process group. Holds this rank's weight rows and channel
    vectors; forward takes replicated fp16 activations [.., K] and returns the full fp16 [.., N]
    on every rank.

    mode: "sym" / "sym_dual" / "asym" / "asym_dual" (activation quantizer and dequant variant).
    Build it from full-size tensors with `from_full` (each rank keeps only its slice)."""

    def __init__(self, mode, n_out, weight, scales_1, zeros_1=None, scales_2=None, zeros_2=None, bias=None,
                 clip_ratio=1.0, group=None, unsharded=False):
        super().__init__()
        self.mode, self.n_out, self.clip_ratio, self.group = mode, n_out, clip_ratio, group
        use_dist = dist.is_initialized() and not unsharded   # unsharded=True: the whole layer on this GPU
        self.world = dist.get_world_size(group) if use_dist else 1
        self.rank = dist.get_rank(group) if use_dist else 0
        self.col_begin, self.col_end = shard_bounds(n_out, self.world, self.rank)
        for name, t in (("weight", weight), ("scales_1", scales_1), ("zeros_1", zeros_1), ("scales_2", scales_2),
                        ("zeros_2", zeros_2), ("bias", bias)):
            if t is not None:
                if t.shape[0] != self.col_end - self.col_begin:
                    raise ValueError(f"{name}: expected {self.col_end - self.col_begin} rows, got {t.shape[0]}")
                self.register_buffer(name, t.contiguous())
            else:
                setattr(self, name, None)
        self._ws = None
        self._peer = None
        self._staging = None
        self._x_dev = self._x_slice = None
        self._w8 = None

    @classmethod
    def from_full(cls, mode, weight, scales_1, zeros_1=None, scales_2=None, zeros_2=None, bias=None, clip_ratio=1.0,
                  group=None):
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        cut = lambda t: None if t is None else shard_rows(t, world, rank)
        return cls(mode, weight.shape[0], cut(weight), cut(scales_1), cut(zeros_1), cut(scales_2), cut(zeros_2), cut(bias),
                   clip_ratio, group)

    def local_forward(self, x2d: torch.Tensor, peer: "PeerOutput" = None):
        """This rank's [M, n_local] block through the fused C-ABI entry point. With `peer`, the
        block is stored into every rank's [M, N] buffer instead of a local tensor."""
        from . import lib as L
        M, K = x2d.shape
        n_local = self.col_end - self.col_begin
        need = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
        if self._ws is None or self._ws.numel() < need or self._ws.device != x2d.device:
            self._ws = torch.empty(need, dtype=torch.uint8, device=x2d.device)
        flat = lambda t: None if t is None else t.reshape(-1)
        if peer is None:
            out = torch.empty((M, n_local), dtype=torch.float16, device=x2d.device)
            epi = L.make_epilogue(self.mode, None, None, flat(self.scales_1), flat(self.zeros_1), flat(self.scales_2),
                                  flat(self.zeros_2), self.bias, col_offset=self.col_begin)
        else:
            out = None
            epi = L.make_epilogue(self.mode, None, None, flat(self.scales_1), flat(self.zeros_1), flat(self.scales_2),
                                  flat(self.zeros_2), self.bias, col_offset=self.col_begin, ldo=self.n_out,
                                  out_peers=peer.column_ptrs(self.col_begin),
                                  out_multicast=peer.multicast_column_ptr(self.col_begin))
        if n_local:
            with torch.cuda.device(x2d.device):
                L.call("duq4_linear_w4a4_from_fp16", L.ptr(x2d), L.ptr(self.weight), M, n_local, K, L.MODES[self.mode],
                       float(self.clip_ratio), ctypes.byref(epi), L.ptr(out), L.ptr(self._ws), self._ws.numel(),
                       L.current_stream())
        return out

    # Layers that see at least this many tokens run on a lazily built int8 re-layout of this rank's weight rows
    # (no unpack in the GEMM); fewer tokens stream the packed rows. See nn/linear.py `weight_prelayout`.
    weight_prelayout = True
    prelayout_min_tokens = 256

    def _weights_for(self, tokens, K):
        """(device pointer argument, w_is_prelaid flag) for the pipeline entry points."""
        from . import lib as L
        if self.weight_prelayout and tokens >= self.prelayout_min_tokens and K % 128 == 0 and self.weight.shape[0] > 0:
            w = self.weight
            key = (w.data_ptr(), w._version)
            if self._w8 is None or self._w8[0] != key:
                w8 = torch.empty((w.shape[0], K), dtype=torch.int8, device=w.device)
                with torch.cuda.device(w.device):
                    L.call("duq4_weight_prelayout_i8", L.ptr(w), w.shape[0], K, L.ptr(w8), L.current_stream())
                self._w8 = (key, w8)
            return L.ptr(self._w8[1]), 1
        return L.ptr(self.weight), 0

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, chunk_rows: int = 0, delivery: str = "columns"):
        """The layer for a job whose activations and result live in HOST memory that every rank maps
        (`SharedHostTensor`; any pinned host tensor when world == 1). PCIe is the scarce resource of such a job,
        NVLink is idle, so every byte crosses PCIe once and in contiguous pieces: rank r uploads rows
        [r*M/G, (r+1)*M/G) of the activations over its own link, the row slices are all-gathered on the devices
        (NCCL over NVLink), and every rank computes its column block row chunk by row chunk. delivery="columns"
        (default): every rank downloads its own [M, N/G] column block into its column slice of `out_host`
        (duq4_linear_w4a4_from_fp16_to_host); the ranks' writes interleave within every host row. delivery="rows":
        the GEMM epilogue stores each row of a chunk into the exchange buffer of the rank that owns the row (an
        all-to-all over NVLink written by the epilogue), a rank barrier completes the chunk and every rank downloads
        the contiguous full-width rows it owns while the next chunk is computed
        (duq4_linear_w4a4_from_fp16_to_host_rows). Measured on 4 and 8 GPUs the two deliver at the same rate: the
        host's aggregate write rate is the limit, not the interleaving.
        One rank: upload, arithmetic and download pipelined by the host-buffer entry point. The result is
        complete once every rank's stream has finished (synchronize, then a host barrier). x_host fp16 [M, K];
        out_host fp16 [M, n_out] row-major."""
        from . import lib as L
        if x_host.is_cuda or out_host.is_cuda:
            raise ValueError("forward_host takes host tensors")
        if x_host.dtype != torch.float16 or out_host.dtype != torch.float16 or not x_host.is_contiguous() or not out_host.is_contiguous():
            raise ValueError("forward_host: contiguous fp16 host tensors expected")
        M, K = x_host.shape
        if tuple(out_host.shape) != (M, self.n_out):
            raise ValueError(f"out_host must be [{M}, {self.n_out}]")
        byte_off, ldo, n_local = host_result_slice(self.n_out, self.world, self.rank)
        if M == 0:
            return
        dev = self.weight.device
        flat = lambda t: None if t is None else t.reshape(-1)
        epi = L.make_epilogue(self.mode, None, None, flat(self.scales_1), flat(self.zeros_1), flat(self.scales_2),
                              flat(self.zeros_2), self.bias, col_offset=self.col_begin, ldo=ldo)
        if self.world == 1:
            need = L.cdll.duq4_linear_host_staging_bytes(M, n_local, K, chunk_rows)
            if self._staging is None or self._staging.numel() < need:
                self._staging = torch.empty(need, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                L.call("duq4_linear_w4a4_from_fp16_host", x_host.data_ptr(), L.ptr(self.weight), M, n_local, K, L.MODES[self.mode],
                       float(self.clip_ratio), ctypes.byref(epi), out_host.data_ptr() + byte_off, chunk_rows, L.ptr(self._staging),
                       self._staging.numel(), L.current_stream())
            return
        # rows of the activations this rank uploads; the gather needs equal slices, so the device copy is padded
        per = -(-M // self.world)
        r0, r1 = min(M, self.rank * per), min(M, (self.rank + 1) * per)
        if self._x_dev is None or self._x_dev.shape != (per * self.world, K):
            self._x_dev = torch.empty((per * self.world, K), dtype=torch.float16, device=dev)
            self._x_slice = torch.zeros((per, K), dtype=torch.float16, device=dev)
        if r1 > r0:
            self._x_slice[: r1 - r0].copy_(x_host[r0:r1], non_blocking=True)
        dist.all_gather_into_tensor(self._x_dev, self._x_slice, group=self.group)
        if delivery == "rows":
            if self._peer is None:
                self._peer = {}
            peer = self._peer.get((M, "host_rows"))
            if peer is None:
                peer = self._peer[(M, "host_rows")] = PeerOutput(M, self.n_out, dev, self.group, use_multicast=False)
            epi = L.make_epilogue(self.mode, None, None, flat(self.scales_1), flat(self.zeros_1), flat(self.scales_2),
                                  flat(self.zeros_2), self.bias, col_offset=self.col_begin, ldo=self.n_out, out_peers=peer.ptrs)
            wptr, prelaid = self._weights_for(M, K) if n_local else (None, 0)
            need = max(256, L.cdll.duq4_linear_pipeline_staging_bytes(0, prelaid, M, max(n_local, 1), K, chunk_rows))
            if self._staging is None or self._staging.numel() < need:
                self._staging = torch.empty(need, dtype=torch.uint8, device=dev)
            epoch = ctypes.c_uint64(peer.epoch)
            try:
                with torch.cuda.device(dev):
                    L.call("duq4_linear_w4a4_from_fp16_to_host_rows", L.ptr(self._x_dev), wptr, prelaid, M, n_local, K, L.MODES[self.mode],
                           float(self.clip_ratio), ctypes.byref(epi), self.col_begin, self.rank, peer._flag_ptrs, ctypes.byref(epoch),
                           peer.barrier_timeout_ns, out_host.data_ptr(), chunk_rows, L.ptr(self._staging), self._staging.numel(),
                           L.current_stream())
            finally:
                peer.epoch = int(epoch.value)
            return
        if delivery != "columns":
            raise ValueError("delivery must be 'rows' or 'columns'")
        if n_local == 0:
            return
        wptr, prelaid = self._weights_for(M, K)
        need = L.cdll.duq4_linear_pipeline_staging_bytes(1, prelaid, M, n_local, K, chunk_rows)
        if self._staging is None or self._staging.numel() < need:
            self._staging = torch.empty(need, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            L.call("duq4_linear_w4a4_from_fp16_to_host", L.ptr(self._x_dev), wptr, prelaid, M, n_local, K, L.MODES[self.mode],
                   float(self.clip_ratio), ctypes.byref(epi), out_host.data_ptr() + byte_off, chunk_rows, L.ptr(self._staging),
                   self._staging.numel(), L.current_stream())

    def forward(self, x: torch.Tensor, gather: str = "nccl"):
        """gather="nccl": compute the local block, then one NCCL all-gather (+ re-layout copy).
        gather="fused": the kernel's epilogue writes the block into every rank's result buffer over
        NVLink: one plain store per peer up to 4 ranks, one multicast store per row segment through the switch from
        8 ranks on, where the switch offers a multicast mapping (measured: a rank's ingress limits the step at 2 and 4
        GPUs and multicast adds the rank's own block to it; at 8 its egress does, which multicast cuts eightfold);
        gather="fused_peer" / "fused_multicast" force one or the other; gather="copy": the epilogue writes the local buffer only
        and copy engines push row chunks to the peers while the next chunk is computed); two device-side barriers
        bracket the launch (peers finished reading
        the previous result / everybody finished writing this one). The returned tensor is a view
        of that shared buffer: it is overwritten by the next fused forward of the same shape."""
        x2d = x.reshape(-1, x.shape[-1]).contiguous()
        if self.world == 1:
            full = self.local_forward(x2d)
        elif gather == "copy":
            # the all-gather on the copy engines: the GEMM of a row chunk writes this rank's block into its own
            # result buffer and 2-D peer copies push the previous chunk to the other ranks meanwhile
            from . import lib as L
            M, K = x2d.shape
            if self._peer is None:
                self._peer = {}
            peer = self._peer.get((M, gather))
            if peer is None:
                peer = self._peer[(M, gather)] = PeerOutput(M, self.n_out, x2d.device, self.group, use_multicast=False)
            n_local = self.col_end - self.col_begin
            flat = lambda t: None if t is None else t.reshape(-1)
            epi = L.make_epilogue(self.mode, None, None, flat(self.scales_1), flat(self.zeros_1), flat(self.scales_2),
                                  flat(self.zeros_2), self.bias, col_offset=self.col_begin, ldo=self.n_out,
                                  out_peers=peer.column_ptrs(self.col_begin))
            wptr, prelaid = self._weights_for(M, K)
            need = L.cdll.duq4_linear_pipeline_staging_bytes(0, prelaid, M, max(n_local, 1), K, 0)
            if self._staging is None or self._staging.numel() < need:
                self._staging = torch.empty(need, dtype=torch.uint8, device=x2d.device)
            peer.barrier()
            if n_local:
                with torch.cuda.device(x2d.device):
                    L.call("duq4_linear_w4a4_from_fp16_to_peers", L.ptr(x2d), wptr, prelaid, M, n_local, K, L.MODES[self.mode],
                           float(self.clip_ratio), ctypes.byref(epi), self.rank, 0, L.ptr(self._staging), self._staging.numel(),
                           L.current_stream())
            peer.barrier()
            full = peer.buf
        elif gather in ("fused", "fused_peer", "fused_multicast"):
            M = x2d.shape[0]
            if self._peer is None:
                self._peer = {}
            peer = self._peer.get((M, gather))
            if peer is None:
                # one shared buffer per token count, kept for the life of the layer: a serving loop that
                # alternates between a few token counts neither re-allocates (a collective rendezvous) nor
                # frees memory a slower rank may still be storing into
                peer = self._peer[(M, gather)] = PeerOutput(M, self.n_out, x2d.device, self.group,
                                                            use_multicast=(gather == "fused_multicast" or (gather == "fused" and self.world >= 8)))
            peer.barrier()
            self.local_forward(x2d, peer)
            peer.barrier()
            full = peer.buf
        else:
            full = gather_columns(self.local_forward(x2d), self.n_out, self.group)
        return full.view(*x.shape[:-1], self.n_out)


# ---------------------------------------------------------------------------------------------
# Row-parallel (K-sharded) layer: the companion of the column-parallel layer for a tensor-parallel
# MLP. The column-parallel gate/up projection leaves every rank with its own block of the hidden
# activations, which is exactly the K-slice the down projection needs: no gather in between.
#
# Bit-exactness with the unsharded layer rests on two facts. (1) Per-token quantizer statistics
# are exact reductions (max / min of fp16 values), so an all-reduce of the per-rank row statistics
# gives every rank the scale (and zero-point) the unsharded quantizer would compute, and each rank
# quantizes its slice with it. (2) The GEMM is an exact integer contraction, so the int32 partial
# accumulators of the K-slices add up to the unsharded accumulators; they are summed across ranks
# BEFORE the fp16 dequant, which then runs once on the totals.


def k_shard_bounds(k_in: int, world: int, rank: int):
    """[begin, end) of the input channels (K) owned by `rank`: contiguous, multiples of 64 channels
    (the GEMM's K granularity) except that trailing ranks may be empty."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if k_in % 64 != 0:
        raise ValueError(f"K = {k_in} is not a multiple of 64")
    per = -(-(k_in // 64) // world) * 64
    b = min(k_in, rank * per)
    return b, min(k_in, b + per)


def _all_reduce_f16(t: torch.Tensor, op, group=None):
    """all-reduce of fp16 values; carried as fp32 (exact for max/min) where the backend has no fp16."""
    if dist.get_backend(group) == "gloo":
        w = t.to(torch.float32)
        dist.all_reduce(w, op=op, group=group)
        return w.to(torch.float16)
    dist.all_reduce(t, op=op, group=group)
    return t


def global_sym_scale(local_absmax: torch.Tensor, clip_ratio: float = 1.0, group=None):
    """Per-token symmetric scale of the FULL row from per-rank abs-max values [M] fp16: the formula of
    the reference's SymQuantizer (qlinear4bit/nn/quantizer.py:10-16) applied to the all-reduced max."""
    amax = _all_reduce_f16(local_absmax.clone(), dist.ReduceOp.MAX, group)
    return (amax / 7).to(torch.float16) * clip_ratio


def global_asym_scale_zeros(local_min: torch.Tensor, local_max: torch.Tensor, group=None):
    """Per-token asymmetric scale and zero-point of the FULL row from per-rank min / max [M] fp16:
    the formula of the reference's AsymQuantizer (qlinear4bit/nn/quantizer.py:24-35)."""
    mn = _all_reduce_f16(local_min.clone(), dist.ReduceOp.MIN, group)
    mx = _all_reduce_f16(local_max.clone(), dist.ReduceOp.MAX, group)
    scale = ((mx - mn) / 15).to(torch.float16)
    zeros = torch.round(-mn / scale).to(torch.float16)
    return scale, zeros


def reduce_partial_accumulators(acc: torch.Tensor, group=None):
    """Sum of the ranks' int32 partial accumulators [M, N], in place on every rank (exact)."""
    dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
    return acc


class RowParallelLinear4bit(torch.nn.Module):
    """One W4A4 layer whose INPUT channels are split over a process group. Holds weight[:, K-slice]
    (packed, [N, Ks/2]) and the full per-output-channel vectors; forward takes this rank's fp16
    activation slice [.., Ks] and returns the full fp16 [.., N] on every rank, bit-identical to the
    unsharded layer.

    mode: "sym" or "asym" (the dual-uniform schemes split the first 10 input channels off, which
    does not commute with a K split; they are rejected)."""

    def __init__(self, mode, k_in, weight, scales, zeros=None, bias=None, clip_ratio=1.0, group=None):
        super().__init__()
        if mode not in ("sym", "asym"):
            raise ValueError(f"row-parallel layer supports 'sym' and 'asym', not {mode!r}")
        if mode == "asym" and zeros is None:
            raise ValueError("asym mode needs weight zero-points")
        self.mode, self.k_in, self.clip_ratio, self.group = mode, k_in, clip_ratio, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k_begin, self.k_end = k_shard_bounds(k_in, self.world, self.rank)
        if weight.shape[1] * 2 != self.k_end - self.k_begin:
            raise ValueError(f"weight: expected {(self.k_end - self.k_begin) // 2} packed columns, got {weight.shape[1]}")
        self.register_buffer("weight", weight.contiguous())
        self.register_buffer("scales", scales.reshape(-1).contiguous())
        self.register_buffer("zeros", None if zeros is None else zeros.reshape(-1).contiguous())
        self.register_buffer("bias", None if bias is None else bias.contiguous())

    @classmethod
    def from_full(cls, mode, weight, scales, zeros=None, bias=None, clip_ratio=1.0, group=None):
        """Build from the unsharded packed weight [N, K/2]; each rank keeps its packed K-slice."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        k_in = weight.shape[1] * 2
        b, e = k_shard_bounds(k_in, world, rank)
        return cls(mode, k_in, weight[:, b // 2: e // 2].contiguous(), scales, zeros, bias, clip_ratio, group)

    def forward(self, x_slice: torch.Tensor, fused: bool = True):
        """fused=True (default with more than one rank): the library's row-parallel pieces -- per-token statistics of
        the slice (one kernel), their all-reduce over the ranks (tiny: one or two fp16 values per token), the fused
        quantizer with the statistics given (one kernel, tensor-core-ready int8 codes), the GEMM whose epilogue stores
        its int32 PARTIAL accumulators straight into the buffer of the rank that owns each block of M/G rows (peer
        stores over NVLink), and after a rank barrier the owner's reduce + single dequant + bias, which stores the fp16
        rows into every rank's result buffer. No int32 all-reduce, no separate quantize / dequant / bias launches.
        fused=False: the same arithmetic composed from the reference-named operators and NCCL (int32 all-reduce)."""
        if fused and self.world > 1 and x_slice.is_cuda:
            return self._forward_fused(x_slice)
        return self._forward_composed(x_slice)

    def _forward_fused(self, x_slice: torch.Tensor):
        import torch.distributed._symmetric_memory as symm
        from . import lib as L
        ks = x_slice.shape[-1]
        M = 1
        for d in x_slice.shape[:-1]:
            M *= int(d)
        x2d = x_slice.reshape(M, ks).contiguous()   # (an empty K slice cannot be reshaped with -1)
        if ks != self.k_end - self.k_begin:
            raise ValueError(f"activation slice has {ks} channels, this rank owns {self.k_end - self.k_begin}")
        N, G, dev = self.weight.shape[0], self.world, x2d.device
        if N % 8 != 0:
            return self._forward_composed(x_slice)   # the owner's pass works on 16-byte row segments
        rpo = -(-M // G)                              # rows per owner
        st = self.__dict__.setdefault("_fstate", {}).get(M)
        if st is None:
            grp = self.group if self.group is not None else dist.group.WORLD
            slabs = symm.empty((G, rpo, N), dtype=torch.int32, device=dev)
            shdl = symm.rendezvous(slabs, grp)
            st = self._fstate[M] = {
                "peer": PeerOutput(M, N, dev, self.group, use_multicast=False),
                "slabs": slabs, "slab_ptrs": [int(p) for p in shdl.buffer_ptrs], "shdl": shdl,
                "stat_a": torch.empty(M, dtype=torch.float16, device=dev), "stat_b": torch.empty(M, dtype=torch.float16, device=dev),
                "a8": torch.empty((M, max(ks, 64)), dtype=torch.int8, device=dev),
                "scale": torch.empty(M, dtype=torch.float16, device=dev), "zeros": torch.empty(M, dtype=torch.float16, device=dev),
            }
        peer, mode_id, asym = st["peer"], L.MODES[self.mode], self.mode == "asym"
        stream = L.current_stream
        with torch.cuda.device(dev):
            # 1. statistics of the slice, reduced over the ranks (exact: max / min of fp16 values)
            if ks:
                L.call("duq4_row_stats", mode_id, L.ptr(x2d), M, ks, L.ptr(st["stat_a"]), L.ptr(st["stat_b"]), stream())
            else:   # an empty slice must not move the global statistics
                st["stat_a"].fill_(float("inf") if asym else 0.0)
                st["stat_b"].fill_(float("-inf"))
            dist.all_reduce(st["stat_a"], op=dist.ReduceOp.MIN if asym else dist.ReduceOp.MAX, group=self.group)
            if asym:
                dist.all_reduce(st["stat_b"], op=dist.ReduceOp.MAX, group=self.group)
            # 2. codes of the slice with the global scale (/ zero-point); every rank derives the same per-token terms
            # (a rank without a K slice still derives the per-token terms: it owns rows of the result)
            L.call("duq4_quantize_i8_from_stats", mode_id, L.ptr(x2d) if ks else None, M, ks, L.ptr(st["stat_a"]), L.ptr(st["stat_b"]),
                   float(self.clip_ratio), L.ptr(st["a8"]) if ks else None, L.ptr(st["scale"]), L.ptr(st["zeros"]), stream())
            # 3. partial accumulators to the owners of the row blocks
            peer.barrier()   # the owners have consumed the previous forward's slabs
            if ks:
                epi = L.make_epilogue("none", acc_owners=st["slab_ptrs"], acc_rows_per_owner=rpo, acc_slot=self.rank)
                L.call("duq4_linear_w4a4_preunpacked", L.ptr(st["a8"]), L.ptr(self.weight), M, N, ks, ctypes.byref(epi), None, None, stream())
            peer.barrier()   # every rank's partial sums have landed
            # 4. this rank's rows: sum of the slabs of the ranks that hold a K slice, one dequant, result to every rank
            n_slabs = sum(1 for r in range(G) if k_shard_bounds(self.k_in, G, r)[1] > k_shard_bounds(self.k_in, G, r)[0])
            row0 = min(M, self.rank * rpo)
            rows = min(M, row0 + rpo) - row0
            if rows:
                epi2 = L.make_epilogue(self.mode, st["scale"], st["zeros"] if asym else None, self.scales, self.zeros if asym else None,
                                       None, None, self.bias, ldo=N, out_peers=peer.ptrs)
                L.call("duq4_reduce_dequant_gather", L.ptr(st["slabs"]), n_slabs, rpo, row0, rows, N, ctypes.byref(epi2), None, stream())
            peer.barrier()   # every owner's rows are in every rank's buffer
        return peer.buf.view(*x_slice.shape[:-1], N)

    def _forward_composed(self, x_slice: torch.Tensor):
        from . import _CUDA
        ks = x_slice.shape[-1]
        M = 1
        for d in x_slice.shape[:-1]:
            M *= int(d)
        x2d = x_slice.reshape(M, ks).contiguous()   # (an empty K slice cannot be reshaped with -1)
        if ks != self.k_end - self.k_begin:
            raise ValueError(f"activation slice has {ks} channels, this rank owns {self.k_end - self.k_begin}")
        n_out = self.weight.shape[0]
        multi = self.world > 1
        if self.mode == "sym":
            if ks:
                amax = torch.max(torch.abs(x2d), dim=-1)[0]
            else:
                amax = torch.zeros(M, dtype=torch.float16, device=x2d.device)
            scale = global_sym_scale(amax, self.clip_ratio, self.group) if multi else (amax / 7).to(torch.float16) * self.clip_ratio
            zeros = None
        else:
            if ks:
                mn, mx = torch.min(x2d, dim=-1)[0], torch.max(x2d, dim=-1)[0]
            else:   # an empty slice must not move the global statistics
                mn = torch.full((M,), float("inf"), dtype=torch.float16, device=x2d.device)
                mx = -mn
            if multi:
                scale, zeros = global_asym_scale_zeros(mn, mx, self.group)
            else:
                scale = ((mx - mn) / 15).to(torch.float16)
                zeros = torch.round(-mn / scale).to(torch.float16)
        if ks:
            q = _CUDA.sym_quant(x2d, scale) if self.mode == "sym" else _CUDA.asym_quant(x2d, scale, zeros)
            acc = _CUDA.matmul(q, self.weight)
        else:
            acc = torch.zeros((M, n_out), dtype=torch.int32, device=x2d.device)
        if multi:
            reduce_partial_accumulators(acc, self.group)
        if self.mode == "sym":
            out = _CUDA.sym_dequant(acc, scale, self.scales, 32)
        else:
            out = _CUDA.asym_dequant(acc, scale, zeros, self.scales, self.zeros, 32)
        if self.bias is not None:
            out = out + self.bias
        return out.view(*x_slice.shape[:-1], n_out)
