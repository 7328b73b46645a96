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

    def __init__(self, device="cuda"):
        self.device = device

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

    def tag_counts(self, tags, n_segments):
        counts = torch.empty(n_segments, dtype=torch.int32, device=tags.device)
        check(lib().xb_tag_counts(xops.ptr(tags), tags.numel(), xops.ptr(counts), n_segments, xops.stream()))
        return counts

    def pool_partial(self, table, rows, vals, counts, dim):
        out = torch.empty((counts.numel(), dim), dtype=torch.float32, device=rows.device)
        g = xops.make_group(table, rows, vals, counts, [dict(udf=capi.XB_UDF_SUM, out=out, col=0)], torch.float32)
        xops.embedding_pool([g])
        return out

    def combine(self, partial, shards, segments, dim, groups, out, seg_len=None, avg=False):
        check(lib().xb_shard_combine(xops.ptr(partial), shards, segments, dim, xops.ptr(seg_len), int(avg), xops.ptr(out),
                                     out.stride(0), groups, xops.dt(out), xops.stream()))
        return out


def sharded_pool(comm, ops, table_shard, dim, ids, values, seg_offsets, groups, out, avg=False):
    """ids/values/seg_offsets: this rank's ids of `groups` feature groups over one row-sharded table,
    laid out group-major (segment = group * rows + sample, rows = samples of this rank);
    out [rows, >= groups*dim] receives the pooled vectors of this rank's samples.
    Returns the per-step byte counts of the two exchanges."""
    W = comm.world
    segments = seg_offsets.numel() - 1
    rows, vals, tags, owner_counts = ops.route(ids, values, seg_offsets, W)
    send_counts = [int(c) for c in owner_counts.cpu()]                       # bucket sizes drive the exchange
    recv_counts = [int(c) for c in comm.exchange_counts(owner_counts).cpu()]
    r_rows = comm.all_to_all_v(rows, send_counts, recv_counts)
    r_vals = comm.all_to_all_v(vals, send_counts, recv_counts)
    r_tags = comm.all_to_all_v(tags, send_counts, recv_counts)
    # segment lengths of every source rank's slice (every rank has the same number of segments)
    counts = []
    pos = 0
    for s in range(W):
        counts.append(ops.tag_counts(r_tags[pos:pos + recv_counts[s]], segments))
        pos += recv_counts[s]
    counts = torch.cat(counts)
    partial = ops.pool_partial(table_shard, r_rows, r_vals, counts, dim)    # [W*segments, dim] fp32
    back = comm.all_to_all_equal(partial)                                    # slice w: from owner w
    seg_len = (seg_offsets[1:] - seg_offsets[:-1]).to(torch.int32) if avg else None
    ops.combine(back, W, segments, dim, groups, out, seg_len, avg)
    return {"routed_bytes": sum(send_counts) * (8 + 4 + 4), "returned_bytes": partial.numel() * 4}
