"""Pooling over row-sharded embedding tables: one process per GPU, ids routed to the
owner of their row and partial pooled vectors returned, both with all-to-all.

`sharded_pool` holds the exchange logic and is backend-agnostic: `ops` does the
device work (GpuShardOps here calls the C-ABI kernels; the CPU tests plug in a
numpy stand-in) and `comm` moves buffers (torch.distributed: NCCL on GPUs, gloo in
the CPU tests). No collective is used outside the two exchange steps.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import capi, ops as xops
from .capi import check, lib


class DistComm:
    """all-to-all over a torch.distributed process group (NCCL or gloo)."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def exchange_counts(self, counts):
        out = torch.empty_like(counts)
        dist.all_to_all_single(out, counts, group=self.group)
        return out

    def all_to_all_v(self, send, send_counts, recv_counts):
        out = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        dist.all_to_all_single(out, send, output_split_sizes=list(recv_counts), input_split_sizes=list(send_counts),
                               group=self.group)
        return out

    def all_to_all_equal(self, send):
        out = torch.empty_like(send)
        dist.all_to_all_single(out, send, group=self.group)
        return out


class GpuShardOps:
    """Device work of the sharded path on the C-ABI kernels."""

    def __init__(self, device="cuda", partial_dtype="f32"):
        """partial_dtype: what the owners return, "f32" (fp32 models, 1e-5 bar) or "f16" (fp16 models: half the
        bytes of the return exchange)."""
        self.device = device
        self.partial_torch = torch.float16 if partial_dtype == "f16" else torch.float32

    def route(self, ids, values, seg_offsets, shards):
        n = ids.numel()
        rows = torch.empty(n, dtype=torch.int64, device=ids.device)
        vals = torch.empty(n, dtype=torch.float32, device=ids.device)
        tags = torch.empty(n, dtype=torch.int32, device=ids.device)
        owner_counts = torch.zeros(shards, dtype=torch.int64, device=ids.device)
        need = int(lib().xb_route_scratch_bytes(n, shards))
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=ids.device)
        check(lib().xb_route_ids(xops.ptr(ids), xops.ptr(values), xops.ptr(seg_offsets), seg_offsets.numel() - 1, n, shards,
                                 xops.ptr(rows), xops.ptr(vals), xops.ptr(tags), xops.ptr(owner_counts), xops.ptr(scratch),
                                 need, xops.stream()))
        return rows, vals, tags, owner_counts

    def route_packed(self, ids, values, seg_offsets, shards):
        """As route, with (segment << 32) | local row in one int64 per id instead of separate rows and tags."""
        n = ids.numel()
        packed = torch.empty(n, dtype=torch.int64, device=ids.device)
        vals = torch.empty(n, dtype=torch.float32, device=ids.device) if values is not None else None
        owner_counts = torch.zeros(shards, dtype=torch.int64, device=ids.device)
        need = int(lib().xb_route_scratch_bytes(n, shards))
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=ids.device)
        check(lib().xb_route_ids(xops.ptr(ids), xops.ptr(values), xops.ptr(seg_offsets), seg_offsets.numel() - 1, n, shards,
                                 xops.ptr(packed), xops.ptr(vals), None, xops.ptr(owner_counts), xops.ptr(scratch),
                                 need, xops.stream()))
        return packed, vals, owner_counts

    def unpack(self, packed):
        rows = torch.empty(packed.numel(), dtype=torch.int32, device=packed.device)
        tags = torch.empty(packed.numel(), dtype=torch.int32, device=packed.device)
        check(lib().xb_unpack_routed(xops.ptr(packed), packed.numel(), xops.ptr(rows), xops.ptr(tags), xops.stream()))
        return rows, tags

    @staticmethod
    def shard_rows(table):
        return table.rows

    def tag_counts(self, tags, n_segments):
        counts = torch.empty(n_segments, dtype=torch.int32, device=tags.device)
        check(lib().xb_tag_counts(xops.ptr(tags), tags.numel(), xops.ptr(counts), n_segments, xops.stream()))
        return counts

    def pool_partial(self, table, rows, vals, counts, dim):
        out = torch.empty((counts.numel(), dim), dtype=torch.float32, device=rows.device)
        g = xops.make_group(table, rows, vals, counts, [dict(udf=capi.XB_UDF_SUM, out=out, col=0)], torch.float32)
        xops.embedding_pool([g])
        return out

    def tag_counts_sources(self, tags, source_counts, n_segments):
        """Segment lengths of every source rank's slice of `tags` (slice lengths `source_counts`, host ints):
        [len(source_counts) * n_segments] int32, one launch."""
        W = len(source_counts)
        counts = torch.empty(W * n_segments, dtype=torch.int32, device=tags.device)
        sc = (C.c_int64 * W)(*source_counts)
        check(lib().xb_tag_counts_sources(xops.ptr(tags), sc, W, xops.ptr(counts), n_segments, xops.stream()))
        return counts

    def pool_partial_tables(self, tables, rows, vals, offsets, sources, table_segments, dim):
        """rows/vals: everything this owner received (source-major, and table-major inside a source);
        offsets [sources * S + 1] int32: where each (source, segment) starts in `rows`, S = sum(table_segments).
        Table t pools the segments [sum(table_segments[:t]), +table_segments[t]) of every source: one pooling
        group per (source, table), all over the same id buffer. Returns [sources * S, dim] fp32."""
        S = sum(table_segments)
        out = torch.empty((sources * S, dim), dtype=self.partial_torch, device=rows.device)
        T = len(tables)
        descs = (C.POINTER(capi.TableDesc) * T)(*[C.pointer(t.desc) for t in tables])
        segs = (C.c_int64 * T)(*table_segments)
        check(lib().xb_shard_pool(descs, segs, T, xops.ptr(rows), xops.dt(rows), rows.numel(), xops.ptr(vals),
                                  xops.ptr(offsets), sources, dim, xops.ptr(out), xops.dt(out), xops.stream()))
        return out

    def combine(self, partial, shards, segments, dim, groups, out, seg_len=None, avg=False):
        check(lib().xb_shard_combine(xops.ptr(partial), xops.dt(partial), shards, segments, dim, xops.ptr(seg_len), int(avg), xops.ptr(out),
                                     out.stride(0), groups, xops.dt(out), xops.stream()))
        return out


def sharded_pool_tables(comm, ops, table_shards, dim, ids, values, seg_offsets, groups, out, avg=False, mark=None):
    """Pooling over several row-sharded tables of one `dim` with ONE routing pass and one pair of exchanges.

    ids[t] / values[t] / seg_offsets[t]: this rank's ids of the `groups[t]` feature groups of table t, laid out
    group-major (segment = group * rows + sample, rows = samples of this rank, the same for every table);
    values[t] may be None (all 1.0) only if it is None for every table. out [rows, >= sum(groups) * dim]
    receives the pooled vectors, table after table. All tables follow the same ownership rule, so their ids
    form one routing problem whose segments are numbered table after table; the owner pools each table's
    segment range against that table's shard. Returns the per-step byte counts of the two exchanges.
    `mark(name)`, when given, is called after each phase (bench.py records a CUDA event there)."""
    mark = mark or (lambda name: None)
    W = comm.world
    T = len(table_shards)
    table_segments = [int(o.numel()) - 1 for o in seg_offsets]
    segments = sum(table_segments)
    if T == 1:
        all_ids, all_vals, all_off = ids[0], values[0], seg_offsets[0]
    else:
        all_ids = torch.cat(list(ids))
        assert all(v is None for v in values) or all(v is not None for v in values)
        all_vals = None if values[0] is None else torch.cat(list(values))
        parts, base = [], 0
        for t in range(T):
            parts.append(seg_offsets[t][:-1] + base if base else seg_offsets[t][:-1])
            base += int(ids[t].numel())
        parts.append(torch.full((1,), base, dtype=seg_offsets[0].dtype, device=seg_offsets[0].device))
        all_off = torch.cat(parts)
    mark("concat")
    # one 8-byte record per id when local rows and segment numbers fit 31 bits, else rows and tags apart
    packed = segments < (1 << 31) and all(ops.shard_rows(t) < (1 << 31) - 1 for t in table_shards)
    if packed:
        recs, vals, owner_counts = ops.route_packed(all_ids, all_vals, all_off, W)
    else:
        rows, vals, tags, owner_counts = ops.route(all_ids, all_vals, all_off, W)
    mark("route")
    both = torch.stack([owner_counts, comm.exchange_counts(owner_counts)]).cpu()   # bucket sizes drive the exchange
    send_counts, recv_counts = [int(c) for c in both[0]], [int(c) for c in both[1]]
    mark("counts")
    if packed:
        r_rows, r_tags = ops.unpack(comm.all_to_all_v(recs, send_counts, recv_counts))
    else:
        r_rows = comm.all_to_all_v(rows, send_counts, recv_counts)
        r_tags = comm.all_to_all_v(tags, send_counts, recv_counts)
    r_vals = comm.all_to_all_v(vals, send_counts, recv_counts) if all_vals is not None else None
    mark("exchange_ids")
    # segment lengths of every source rank's slice (every rank has the same number of segments), then where
    # every (source, segment) starts in the received buffer
    offsets = torch.zeros(W * segments + 1, dtype=torch.int32, device=r_tags.device)
    torch.cumsum(ops.tag_counts_sources(r_tags, recv_counts, segments), 0, dtype=torch.int32, out=offsets[1:])
    mark("offsets")
    partial = ops.pool_partial_tables(table_shards, r_rows, r_vals, offsets, W, table_segments, dim)   # [W*segments, dim] fp32
    mark("pool")
    back = comm.all_to_all_equal(partial)                                    # slice w: from owner w
    mark("exchange_partials")
    seg_len = (all_off[1:] - all_off[:-1]).to(torch.int32) if avg else None
    ops.combine(back, W, segments, dim, sum(groups), out, seg_len, avg)
    mark("combine")
    per_id = (8 if packed else 12) + (4 if all_vals is not None else 0)
    return {"routed_bytes": sum(send_counts) * per_id, "returned_bytes": partial.numel() * partial.element_size()}


def sharded_pool(comm, ops, table_shard, dim, ids, values, seg_offsets, groups, out, avg=False):
    """One table: ids/values/seg_offsets are this rank's ids of `groups` feature groups (group-major segments),
    out [rows, >= groups*dim] receives the pooled vectors of this rank's samples."""
    return sharded_pool_tables(comm, ops, [table_shard], dim, [ids], [values], [seg_offsets], [groups], out, avg)


class ShardContext:
    """One rank's context of the sharded step that runs entirely behind the C ABI (xb_shard_ctx_create /
    xb_sharded_pool): buffers allocated once, NCCL called from inside the library, no host synchronisation in a
    step. `tables` are this rank's shards (ops.Table with identity keys), `table_segments[t]` the segments of
    table t per step on this rank. With world > 1 every rank calls this with the same `unique_id`
    (ShardContext.unique_id() on one rank, handed to the others by any transport)."""

    def __init__(self, rank, world, tables, table_segments, dim, max_ids, partial_dtype="f16", capacity_factor=2.0,
                 unique_id=None):
        T = len(tables)
        self._tables = tables
        self._descs = (C.POINTER(capi.TableDesc) * T)(*[C.pointer(t.desc) for t in tables])
        self._segs = (C.c_int64 * T)(*table_segments)
        cfg = capi.ShardConfig()
        cfg.rank, cfg.world, cfg.dim, cfg.n_tables = rank, world, dim, T
        cfg.tables, cfg.table_segments = C.cast(self._descs, C.c_void_p), C.cast(self._segs, C.c_void_p)
        cfg.max_ids = max_ids
        cfg.partial_dtype = capi.XB_F16 if partial_dtype == "f16" else capi.XB_F32
        cfg.capacity_factor = capacity_factor
        self.h = C.c_void_p()
        self.segments, self.dim, self.world = sum(table_segments), dim, world
        self._id = unique_id
        check(lib().xb_shard_ctx_create(C.byref(self.h), unique_id, C.byref(cfg)))

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(128)
        check(lib().xb_shard_unique_id(buf))
        return buf.raw

    def pool(self, ids, seg_offsets, groups, out):
        """ids int64 [n], seg_offsets int32 [segments + 1] (all tables, group-major), out [rows, >= groups * dim]."""
        check(lib().xb_sharded_pool(self.h, xops.ptr(ids), xops.ptr(seg_offsets), ids.numel(), groups, 0, xops.ptr(out),
                                    out.stride(0), xops.dt(out), xops.stream()))
        return out

    def begin(self, ids, seg_offsets):
        """First half of a step on the current stream: bucket the ids and exchange them (see xb_sharded_pool_begin)."""
        check(lib().xb_sharded_pool_begin(self.h, xops.ptr(ids), xops.ptr(seg_offsets), ids.numel(), xops.stream()))

    def finish(self, groups, out):
        """Second half of the oldest begun step on the current stream: pooling, exchange of partial sums, combine."""
        check(lib().xb_sharded_pool_finish(self.h, groups, 0, xops.ptr(out), out.stride(0), xops.dt(out), xops.stream()))
        return out

    def pool_stage(self):
        """Middle part of the oldest begun step on the current stream: owner pooling and exchange of the partial sums."""
        check(lib().xb_sharded_pool_pool(self.h, xops.stream()))

    def combine(self, groups, out):
        """Last part of the oldest pooled step on the current stream."""
        check(lib().xb_sharded_pool_combine(self.h, groups, 0, xops.ptr(out), out.stride(0), xops.dt(out), xops.stream()))
        return out

    def overflow(self):
        """After a stream synchronisation: True when a step since the last call dropped ids (bucket capacity)."""
        f = C.c_int32(0)
        check(lib().xb_shard_ctx_status(self.h, C.byref(f)))
        return bool(f.value)

    @property
    def bucket_capacity(self):
        return int(lib().xb_shard_ctx_bucket_capacity(self.h))

    @property
    def device_bytes(self):
        return int(lib().xb_shard_ctx_device_bytes(self.h))

    PHASES = ("bucket_ids", "exchange_ids", "lengths_offsets", "pool", "exchange_partials", "combine")

    def profile(self, enable=True):
        """Record events at the phase boundaries of every pool() call from now on (off by default)."""
        check(lib().xb_shard_ctx_profile(self.h, int(enable)))

    def phase_ms(self):
        """Milliseconds of the six phases of the last profiled pool() call; synchronise the stream first."""
        import ctypes as C
        buf = (C.c_float * 6)()
        check(lib().xb_shard_ctx_phase_ms(self.h, C.cast(buf, C.c_void_p)))
        return dict(zip(self.PHASES, (float(x) for x in buf)))

    def close(self):
        if self.h:
            lib().xb_shard_ctx_destroy(self.h)
            self.h = C.c_void_p()
