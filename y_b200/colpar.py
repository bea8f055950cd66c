"""Column-parallel (N-sharded) use of the FP8 GEMM across the GPUs of one node.

Rank r owns the weight columns [r*N_s, (r+1)*N_s) as a K-major e4m3 shard; the
activations are replicated and every rank runs the RMSNorm->e4m3 prologue itself
(cheaper than a broadcast). The data path has no collective. Two exchanges exist
around it: one scalar all-reduce(MAX) of the weight amax when the shards are
quantised, so the sharded result is bit-identical to the unsharded one, and an
optional all-gather of the bf16 output shards. Works on any torch.distributed
backend (NCCL on GPUs; gloo in the CPU tests of the host logic).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_total: int, world: int, rank: int, multiple: int = 16) -> tuple[int, int]:
    """Column range of `rank`. Shards are equal and a multiple of `multiple` columns
    (16 keeps rows of every shard 16-byte aligned for any element type)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n_total % world != 0:
        raise ValueError(f"N={n_total} does not divide over {world} ranks")
    n_s = n_total // world
    if n_s % multiple != 0:
        raise ValueError(f"shard width {n_s} is not a multiple of {multiple}")
    return rank * n_s, (rank + 1) * n_s


def agree_amax(local_amax: torch.Tensor, group=None) -> torch.Tensor:
    """Global max of the per-shard amax (in place); one scale for the whole weight."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_amax, op=dist.ReduceOp.MAX, group=group)
    return local_amax


def gather_columns(c_local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """All-gather of the output shards. Returns [world, M, N_s] (rank-major: the
    layout a contiguous all-gather produces; `assemble` gives row-major [M, N])."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    m, n_s = c_local.shape
    if out is None:
        out = torch.empty((world, m, n_s), dtype=c_local.dtype, device=c_local.device)
    if world == 1:
        out[0].copy_(c_local)
        return out
    if out.shape != (world, m, n_s):
        raise ValueError(f"gather buffer has shape {tuple(out.shape)}, want {(world, m, n_s)}")
    dist.all_gather_into_tensor(out.view(world * m, n_s), c_local.contiguous(), group=group)
    return out


def assemble(gathered: torch.Tensor) -> torch.Tensor:
    """[world, M, N_s] -> row-major [M, world * N_s]."""
    world, m, n_s = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * n_s)


class _RawOut:
    """A device address with a shape and dtype, accepted where the operator layer takes `out`."""

    def __init__(self, ptr: int, shape, dtype, device):
        self._ptr, self.shape, self.dtype, self.device = ptr, tuple(shape), dtype, device

    def data_ptr(self) -> int:
        return self._ptr


class GatheredOutput:
    """The gathered output [world, M, N_s] of a column-parallel GEMM, filled by the GEMM's own
    epilogue instead of a collective: every rank allocates the buffers in memory its peers can
    map (CUDA IPC through the library), and each rank's GEMM stores its shard into slot `rank`
    of every rank's current buffer with plain NVLink stores. `barrier()` orders the ranks on
    the current stream; after it every rank may read its current buffer.

    Reuse. A peer may start the next step's GEMM (and with it the stores into this rank's
    memory) as soon as its own `barrier()` has completed, which does not wait for this rank's
    reads. So there are `buffers` (>= 2) buffers used in turn: `advance()` moves every rank to
    the next one before the next step, and a buffer is written again only `buffers` steps
    later, i.e. after at least one further `barrier()` that every rank enters only once its
    reads of that buffer (enqueued on the same stream before the barrier) are done. The rule
    for the caller: read the current buffer on the stream the step runs on, before the next
    step's `barrier()` is enqueued there, and call `advance()` on every rank between steps.
    With `buffers=1` the caller has to put a second `barrier()` after its reads itself.
    """

    def __init__(self, m: int, n_shard: int, dtype=torch.bfloat16, group=None, buffers: int = 2):
        import ctypes as C

        from ._lib import check, lib

        if buffers < 1:
            raise ValueError("buffers must be >= 1")
        self._lib, self._check, self._C = lib, check, C
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.n_shard, self.dtype = m, n_shard, dtype
        self.buffers, self.current = buffers, 0
        self.slot_bytes = m * n_shard * torch.empty((), dtype=dtype).element_size()
        self.buffer_bytes = self.slot_bytes * self.world
        base = C.c_void_p()
        check(lib.y_b200_peer_alloc(self.buffer_bytes * buffers, C.byref(base)))
        self.base = base.value
        handle = C.create_string_buffer(64)
        check(lib.y_b200_peer_export(self.base, handle))
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_bases = {}
        for r, h in enumerate(handles):
            if r == self.rank or h is None:
                continue
            ptr = C.c_void_p()
            check(lib.y_b200_peer_open(h, C.byref(ptr)))
            self.peer_bases[r] = ptr.value
        self._token = torch.zeros(1, device="cuda")

    def advance(self) -> None:
        """Switch to the next buffer (every rank, between steps)."""
        self.current = (self.current + 1) % self.buffers

    def _buffer_offset(self) -> int:
        return self.current * self.buffer_bytes

    def local_slot(self) -> int:
        """Device address of this rank's slot in its own current buffer (the GEMM's `c`)."""
        return self.base + self._buffer_offset() + self.rank * self.slot_bytes

    def replica_slots(self) -> list[int]:
        """Device addresses of this rank's slot in every peer's current buffer (the GEMM's replicas)."""
        off = self._buffer_offset() + self.rank * self.slot_bytes
        return [b + off for _, b in sorted(self.peer_bases.items())]

    def barrier(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)  # stream-ordered on every rank

    def to_host(self) -> torch.Tensor:
        """Copy of the current gathered buffer as a CPU tensor [world, M, N_s] (for checks)."""
        out = torch.empty((self.world, self.m, self.n_shard), dtype=self.dtype)
        torch.cuda.synchronize()
        self._check(self._lib.y_b200_peer_read(out.data_ptr(), self.base + self._buffer_offset(), self.buffer_bytes))
        return out

    def close(self) -> None:
        """Unmap the peers' buffers, wait for every rank to have done so, then free this one."""
        for b in self.peer_bases.values():
            self._check(self._lib.y_b200_peer_close(b))
        self.peer_bases = {}
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        if self.base:
            self._check(self._lib.y_b200_peer_free(self.base))
            self.base = 0


class ColumnParallelFp8Linear:
    """One rank's shard of `C = rmsnorm(X; gamma, eps) -> e4m3, then FP8 GEMM with the
    pre-quantised weight shard -> bf16`, with a device path and a pipelined host path.

    `forward(x)` runs the step on the current stream (x on the device). `submit_host`
    takes pinned host buffers: the host->device copy of step i+1, the kernels of step
    i and the device->host copy of step i-1 run on three streams at the same time, so
    the two directions of the host link and the GPU overlap; `drain` makes the current
    stream wait for everything submitted. On one rank this is the library's own
    `y_colpar_submit_host` / `y_colpar_drain` (the C entry a non-Python host binds), and this
    class only holds the handle. With more than one rank the activations are the same on
    every rank, so each rank copies only its 1/world of the rows from the host and the ranks
    all-gather the rest over NVLink on the copy-in stream (every rank must call `submit_host`
    the same number of times); that exchange is torch.distributed's, so this path keeps its
    streams here. Buffers are reused round-robin over `depth` slots; a host output buffer may
    be read after `drain` (or after the event `submit_host` returns has completed).
    """

    def __init__(self, bqt: torch.Tensor, scale_b, gamma: torch.Tensor, eps: float, m: int, depth: int = 2,
                 group=None):
        from . import quant as q

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0

        self._q = q
        self.bqt, self.scale_b, self.gamma, self.eps = bqt, scale_b, gamma, float(eps)
        self.n_shard, self.k = bqt.shape
        self.m, self.depth = m, depth
        dev = bqt.device
        ws_bytes = int(q.lib.y_b200_rmsnorm_workspace_bytes(m))
        self._ws = [torch.empty(ws_bytes, dtype=torch.uint8, device=dev) for _ in range(depth)]
        self._aq = [torch.empty((m, self.k), dtype=torch.uint8, device=dev) for _ in range(depth)]
        self._x = self._c = None  # host-path staging, allocated on first use
        self._streams = None
        self._count = 0
        self._handle = None       # y_colpar handle of the single-rank host path

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, slot: int = 0,
                gathered: "GatheredOutput | None" = None) -> torch.Tensor:
        """With `gathered`, the GEMM's epilogue also stores the shard into this rank's slot on
        every peer (call `gathered.barrier()` before reading); `out` is then ignored."""
        q = self._q
        aq, sa = q.rmsnorm_quantize_fp8(x, self.gamma, self.eps, workspace=self._ws[slot], out=self._aq[slot])
        if gathered is None:
            return q.gemm_fp8_codes(aq, self.bqt, sa, self.scale_b, out_dtype=torch.bfloat16, out=out)
        return q.gemm_fp8_codes(aq, self.bqt, sa, self.scale_b, out_dtype=torch.bfloat16,
                                out=_RawOut(gathered.local_slot(), (self.m, self.n_shard), torch.bfloat16, x.device),
                                replicas=gathered.replica_slots())

    # ---- single rank: the library's pipelined host path -------------------------------------
    def _c_handle(self):
        if self._handle is None:
            q = self._q
            sb = self.scale_b
            if not isinstance(sb, torch.Tensor):
                sb = torch.tensor([float(sb)], dtype=torch.float32, device=self.bqt.device)
            self._scale_b_dev = sb  # kept alive: the handle holds its address
            h = q.lib.y_colpar_create(self.bqt.data_ptr(), sb.data_ptr(), self.gamma.data_ptr(), self.eps, self.m, self.k,
                                      self.n_shard, self.depth)
            if not h:
                from ._lib import YB200Error, last_error
                raise YB200Error(-4, last_error())
            self._handle = h
        return self._handle

    def close(self) -> None:
        if self._handle is not None:
            self._q.lib.y_colpar_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- several ranks: the same pipeline with the row exchange on the copy-in stream ---------
    def _host_state(self):
        if self._streams is None:
            dev = self.bqt.device
            self._streams = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
            self._x = [torch.empty((self.m, self.k), dtype=torch.float16, device=dev) for _ in range(self.depth)]
            self._c = [torch.empty((self.m, self.n_shard), dtype=torch.bfloat16, device=dev)
                       for _ in range(self.depth)]
            self._ev = [[torch.cuda.Event() for _ in range(self.depth)] for _ in range(3)]
            for kind in self._ev:
                for e in kind:
                    e.record()
        return self._streams

    def _shares_rows(self) -> bool:
        return self.world > 1 and self.m % self.world == 0

    def submit_host(self, x_host: torch.Tensor, c_host: torch.Tensor):
        """Enqueues one step with pinned host input and output. Returns an event that completes
        with the copy-out (several ranks) or None (one rank: use `drain`)."""
        if not (x_host.is_pinned() and c_host.is_pinned()):
            raise ValueError("submit_host takes pinned host tensors")
        if self.world == 1:
            from ._lib import check
            check(self._q.lib.y_colpar_submit_host(self._c_handle(), x_host.data_ptr(), c_host.data_ptr(),
                                                   torch.cuda.current_stream(self.bqt.device).cuda_stream))
            return None
        s_in, s_cmp, s_out = self._host_state()
        i = self._count % self.depth
        self._count += 1
        in_done, cmp_done, out_done = self._ev[0][i], self._ev[1][i], self._ev[2][i]
        start = torch.cuda.Event()
        start.record()  # work submitted earlier on the caller's stream (e.g. filling x_host) comes first
        with torch.cuda.stream(s_in):
            s_in.wait_event(start)
            s_in.wait_event(cmp_done)  # the kernels that last read this slot's x are done
            if self._shares_rows():
                rows = self.m // self.world
                mine = slice(self.rank * rows, (self.rank + 1) * rows)
                self._x[i][mine].copy_(x_host[mine], non_blocking=True)
                # The exchange of the row blocks rides on the copy-in stream, so it overlaps the
                # kernels of the step before; in place: this rank's rows already sit where the
                # gather puts them.
                dist.all_gather_into_tensor(self._x[i], self._x[i][mine], group=self.group)
            else:
                self._x[i].copy_(x_host, non_blocking=True)
            in_done.record()
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(in_done)
            s_cmp.wait_event(out_done)  # the copy that last read this slot's c is done
            self.forward(self._x[i], out=self._c[i], slot=i)
            cmp_done.record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(cmp_done)
            c_host.copy_(self._c[i], non_blocking=True)
            out_done.record()
        return out_done

    def host_api(self) -> str:
        """The call a step with host buffers goes through."""
        if self.world == 1:
            return "y_colpar_submit_host / y_colpar_drain (C ABI; 3-stream pipeline inside the library)"
        return ("y_b200.colpar.ColumnParallelFp8Linear.submit_host (3-stream pipeline; rows of X shared by "
                "torch.distributed all-gather on the copy-in stream)")

    def host_bytes_per_step(self) -> tuple[int, int]:
        """(host->device, device->host) bytes this rank moves per `submit_host`."""
        share = self.world if self._shares_rows() else 1
        return self.m * self.k * 2 // share, self.m * self.n_shard * 2

    def drain(self) -> None:
        if self.world == 1:
            if self._handle is not None:
                from ._lib import check
                check(self._q.lib.y_colpar_drain(self._handle, torch.cuda.current_stream(self.bqt.device).cuda_stream))
            return
        if self._streams is None:
            return
        cur = torch.cuda.current_stream(self.bqt.device)
        for kind in self._ev:
            for e in kind:
                cur.wait_event(e)
