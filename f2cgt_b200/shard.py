"""Row-sharded compressed table on one NVSwitch box: rank r owns rows [r*rows_per_rank, (r+1)*rows_per_rank).

Two ways to aggregate a block whose source rows live on other GPUs:

* ``ShardedTable.fetch(ids)`` - the exchange the reference never needed (it keeps one pinned replica per machine,
  examples/load_dataset.py:63-85): ids are bucketed by owner, exchanged, the owners gather their rows, and the rows
  are exchanged back, each exchange one NCCL ``all_to_all_single`` with per-peer split sizes (over gloo on CPU,
  which is how the tests cover the host logic, the same exchange is a group of point-to-point operations).
  The fused kernel then runs on the fetched, block-local rows.
* ``PeerTable`` - every rank maps the other ranks' shards through CUDA IPC (``f2c_shard_create`` / ``f2c_shard_open``)
  and the fused kernel reads remote rows itself with ordinary loads over NVLink (``f2c_sq_spmm_csr_peer``): no
  collective, no host synchronisation.

Host logic only; all arithmetic is in the CUDA library.
"""
import torch
import torch.distributed as dist


def rows_per_rank(n_rows, world):
    """Rows per shard: ceil(n_rows / world), at least 2 (the kernels divide by it with a multiply-high that needs >= 2);
    the last shards of a small or uneven table may be short or empty."""
    return max(2, (n_rows + world - 1) // world)


def shard_bounds(n_rows, world, rank):
    rpr = rows_per_rank(n_rows, world)
    return min(rank * rpr, n_rows), min((rank + 1) * rpr, n_rows)


def bucket_by_owner(ids, rpr, world):
    """Stable bucketing of global row ids by owning rank.

    Returns (order, sorted_ids, counts): ids[order] == sorted_ids is grouped by owner, counts[r] ids go to rank r."""
    owner = torch.div(ids, rpr, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world)[:world]
    return order, ids[order], counts


def _exchange(send, send_counts, recv_counts, group):
    """Variable-size all-to-all of the leading dimension: ``all_to_all_single`` with split sizes on CUDA tensors, one
    group of point-to-point operations on CPU tensors."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    recv = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
    if send.is_cuda:  # NCCL: one all-to-all with per-peer split sizes (gloo, which the CPU tests run on, has none: see below)
        dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=[int(c) for c in recv_counts],
                               input_split_sizes=[int(c) for c in send_counts], group=group)
        return recv
    s_off = [0]
    r_off = [0]
    for r in range(world):
        s_off.append(s_off[-1] + int(send_counts[r]))
        r_off.append(r_off[-1] + int(recv_counts[r]))
    ops = []
    for r in range(world):
        if r == rank:
            recv[r_off[r]:r_off[r + 1]].copy_(send[s_off[r]:s_off[r + 1]])
            continue
        if recv_counts[r] > 0:
            ops.append(dist.P2POp(dist.irecv, recv[r_off[r]:r_off[r + 1]], dist.get_global_rank(group, r) if group else r, group))
        if send_counts[r] > 0:
            ops.append(dist.P2POp(dist.isend, send[s_off[r]:s_off[r + 1]].contiguous(), dist.get_global_rank(group, r) if group else r, group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return recv


class ShardedTable:
    """One rank's shard of a [n_rows, row_width] table plus the row fetch over the process group."""

    def __init__(self, local_rows, n_rows, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_rows = int(n_rows)
        self.rpr = rows_per_rank(self.n_rows, self.world)
        lo, hi = shard_bounds(self.n_rows, self.world, self.rank)
        if local_rows.shape[0] != hi - lo:
            raise ValueError(f"rank {self.rank} must hold rows [{lo}, {hi}) - got {local_rows.shape[0]} rows")
        self.local = local_rows
        self.lo = lo

    def plan(self, ids, check=True):
        """Everything about a fetch that depends only on the ids (can be computed when the block is sampled):
        bucketing, the count exchange and the id exchange.  Returns a dict consumed by ``fetch_rows``.
        ``check=False`` skips the range test of the ids and its host read (ids that come straight from the sampler)."""
        if check and ids.numel():
            lo_hi = torch.stack(torch.aminmax(ids)).tolist()  # one host read for both bounds
            if lo_hi[0] < 0 or lo_hi[1] >= self.n_rows:
                raise IndexError("row id outside the table")
        order, sorted_ids, counts = bucket_by_owner(ids, self.rpr, self.world)
        if ids.is_cuda:  # one small all-to-all of the counts on the device, one host read for both directions
            got = torch.empty_like(counts)
            dist.all_to_all_single(got, counts.contiguous(), group=self.group)
            both = torch.stack([counts, got]).to("cpu").tolist()
            send_counts, recv_counts = both[0], both[1]
        else:
            send_counts = counts.to("cpu").tolist()
            all_counts = [None] * self.world
            dist.all_gather_object(all_counts, send_counts, group=self.group)
            recv_counts = [all_counts[r][self.rank] for r in range(self.world)]
        wanted = _exchange(sorted_ids, send_counts, recv_counts, self.group)  # ids other ranks want from this shard
        # position[j] = where the row of ids[j] lands in the buffer the exchange fills (rows arrive grouped by owner)
        position = torch.empty_like(order)
        position[order] = torch.arange(order.numel(), dtype=order.dtype, device=order.device)
        return dict(order=order, position=position, send_counts=send_counts, recv_counts=recv_counts, local_index=wanted - self.lo)

    def fetch_rows(self, plan, ordered=True):
        """Owner-side gather + row exchange.  ``ordered=True``: the rows in the order of the ids given to ``plan``.
        ``ordered=False``: the rows as they arrive (grouped by owner) - the row of ``ids[j]`` is row ``plan["position"][j]``;
        a caller that renumbers its block indices through ``position`` once (indices are 8 bytes, rows 16 .. 128) saves a
        pass over every fetched table."""
        rows = self.local.index_select(0, plan["local_index"])
        got = _exchange(rows, plan["recv_counts"], plan["send_counts"], self.group)
        if not ordered:
            return got
        out = torch.empty_like(got)
        out[plan["order"]] = got
        return out

    def fetch(self, ids):
        return self.fetch_rows(self.plan(ids))


class _LibraryShards:
    """Shard memory through the library: f2c_shard_create / open / close / free (CUDA IPC)."""

    def create(self, rows):
        import ctypes
        from ._lib import lib, check
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        check(lib.f2c_shard_create(rows.data_ptr(), rows.numel() * rows.element_size(), ctypes.byref(own), handle,
                                   torch.cuda.current_stream(rows.device).cuda_stream))
        return own.value, bytes(handle)

    def open(self, handle):
        import ctypes
        from ._lib import lib, check
        ptr = ctypes.c_void_p()
        check(lib.f2c_shard_open((ctypes.c_ubyte * 64).from_buffer_copy(handle), ctypes.byref(ptr)))
        return ptr.value

    def close(self, ptr):
        import ctypes
        from ._lib import lib, check
        check(lib.f2c_shard_close(ctypes.c_void_p(ptr)))

    def free(self, ptr):
        import ctypes
        from ._lib import lib, check
        check(lib.f2c_shard_free(ctypes.c_void_p(ptr)))


class PeerTable:
    """Shards of all ranks mapped into this process through CUDA IPC (plain peer mappings, no multicast).

    The local rows are copied once into an allocation of their own that the library exports
    (``f2c_shard_create``); every other rank opens the handle while ITS GPU is the current device
    (``f2c_shard_open``), which maps the memory into that GPU's address space with peer access.
    ``pointers[r]`` is the device address of rank r's shard as seen from this rank.  Construct and ``close`` it
    collectively: every rank closes its mappings before any owner frees its shard.

    A failure on any rank (allocation, export, mapping) is gathered and raised on EVERY rank after the collectives, so no
    rank is left waiting in one.  An empty shard (the last ranks of a small or uneven table) is exported as one zero row.
    ``backend`` replaces the library's shard calls (tests inject failures on CPU ranks with it)."""

    def __init__(self, local_rows, n_rows, group=None, backend=None):
        self.backend = backend or _LibraryShards()
        if backend is None and (not local_rows.is_cuda or not local_rows.is_contiguous() or local_rows.dim() != 2):
            raise ValueError("local_rows must be a contiguous 2-D CUDA tensor")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_rows = int(n_rows)
        self.rpr = rows_per_rank(self.n_rows, self.world)
        lo, hi = shard_bounds(self.n_rows, self.world, self.rank)
        if local_rows.shape[0] != hi - lo:
            raise ValueError(f"rank {self.rank} must hold rows [{lo}, {hi}) - got {local_rows.shape[0]} rows")
        self.device = local_rows.device
        self.dtype = local_rows.dtype
        self.row_width = int(local_rows.shape[1])
        self.nbytes = local_rows.numel() * local_rows.element_size()
        self._own = None
        self._opened = []
        self.pointers = []
        self.shard_bytes = []
        guard = torch.cuda.device(self.device) if self.device.type == "cuda" else _NoGuard()
        with guard:
            err, handle = None, b""
            try:
                export = local_rows if self.nbytes > 0 else torch.zeros((1, max(self.row_width, 1)), dtype=self.dtype, device=self.device)
                self._own, handle = self.backend.create(export)
            except Exception as e:  # noqa: BLE001
                err = f"rank {self.rank}: {e}"
            metas = [None] * self.world
            dist.all_gather_object(metas, (handle, self.nbytes, err), group=self.group)
            failed = [m[2] for m in metas if m[2] is not None]
            if not failed:
                for r, (h, nbytes, _) in enumerate(metas):
                    self.shard_bytes.append(nbytes)
                    if r == self.rank:
                        self.pointers.append(self._own)
                        continue
                    try:
                        ptr = self.backend.open(h)
                    except Exception as e:  # noqa: BLE001
                        err = f"rank {self.rank} opening shard {r}: {e}"
                        break
                    self._opened.append(ptr)
                    self.pointers.append(ptr)
            opened = [None] * self.world  # second round: did every rank map every shard?
            dist.all_gather_object(opened, err, group=self.group)
            failed += [m for m in opened if m is not None and m not in failed]
            if failed:
                self._release()
                raise RuntimeError("PeerTable: " + "; ".join(failed))
        dist.barrier(group=self.group)

    def _release(self):
        """Collective: unmap the other ranks' shards, then free the local one (errors while cleaning up are dropped)."""
        for ptr in self._opened:
            try:
                self.backend.close(ptr)
            except Exception:  # noqa: BLE001
                pass
        self._opened = []
        dist.barrier(group=self.group)
        if self._own:
            try:
                self.backend.free(self._own)
            except Exception:  # noqa: BLE001
                pass
        self._own = None
        self.pointers = []

    def read(self, r, byte_offset, nbytes):
        """Bytes [byte_offset, byte_offset + nbytes) of rank r's shard as a uint8 tensor on this GPU (copy engine)."""
        from ._lib import lib, check
        if byte_offset < 0 or byte_offset + nbytes > self.shard_bytes[r]:
            raise IndexError("range outside the shard")
        out = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            check(lib.f2c_shard_copy(out.data_ptr(), self.pointers[r] + byte_offset, nbytes,
                                     torch.cuda.current_stream(self.device).cuda_stream))
        return out

    def close(self):
        """Collective: unmap the other ranks' shards, then free the local one."""
        if self._own is None:
            return
        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                torch.cuda.synchronize(self.device)
                self._release()
        else:
            self._release()


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
