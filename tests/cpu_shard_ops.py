"""CPU stand-in for the device side of the sharded pooling path (numpy + the CPU oracle).
TEST INFRASTRUCTURE: lets the exchange logic of x-deeplearning_b200/sharded.py run under gloo."""
import numpy as np
import torch

import orc


class CpuShardOps:
    def route(self, ids, values, seg_offsets, shards):
        idn = ids.numpy()
        owner, local = orc.route(idn, shards)
        order = np.argsort(owner, kind="stable")
        tags = np.searchsorted(seg_offsets.numpy(), np.arange(len(idn)), side="right") - 1
        counts = np.bincount(owner, minlength=shards).astype(np.int64)
        v = values.numpy() if values is not None else np.ones(len(idn), np.float32)
        return (torch.from_numpy(local[order]), torch.from_numpy(v[order].astype(np.float32)),
                torch.from_numpy(tags[order].astype(np.int32)), torch.from_numpy(counts))

    def route_packed(self, ids, values, seg_offsets, shards):
        rows, vals, tags, counts = self.route(ids, values, seg_offsets, shards)
        r = np.minimum(rows.numpy().astype(np.uint64), np.uint64(0x7fffffff))
        packed = (tags.numpy().astype(np.uint64) << np.uint64(32)) | r
        return torch.from_numpy(packed.astype(np.int64)), (vals if values is not None else None), counts

    def unpack(self, packed):
        v = packed.numpy().astype(np.uint64)
        return (torch.from_numpy((v & np.uint64(0xffffffff)).astype(np.int32)),
                torch.from_numpy((v >> np.uint64(32)).astype(np.int32)))

    @staticmethod
    def shard_rows(table):
        return len(table)

    def tag_counts(self, tags, n_segments):
        return torch.from_numpy(np.bincount(tags.numpy(), minlength=n_segments).astype(np.int32))

    def tag_counts_sources(self, tags, source_counts, n_segments):
        out, pos = [], 0
        for n in source_counts:
            out.append(self.tag_counts(tags[pos:pos + n], n_segments))
            pos += n
        return torch.cat(out)

    def pool_partial(self, table, rows, vals, counts, dim):
        out = np.zeros((counts.numel(), dim), np.float32)
        orc.embedding_pool(table, rows.numpy(), vals.numpy(), counts.numpy(), [dict(udf=0, out=out, col=0)])
        return torch.from_numpy(out)

    def pool_partial_tables(self, tables, rows, vals, offsets, sources, table_segments, dim):
        S = sum(table_segments)
        off = offsets.numpy()
        out = np.zeros((sources * S, dim), np.float32)
        r = rows.numpy()
        v = vals.numpy() if vals is not None else np.ones(len(r), np.float32)
        for s in range(sources):
            lo = s * S
            for table, n in zip(tables, table_segments):
                a, b = int(off[lo]), int(off[lo + n])
                counts = (off[lo + 1:lo + n + 1] - off[lo:lo + n]).astype(np.int32)
                part = np.zeros((n, dim), np.float32)
                orc.embedding_pool(table, r[a:b], v[a:b], counts, [dict(udf=0, out=part, col=0)])
                out[lo:lo + n] = part
                lo += n
        return torch.from_numpy(out)

    def combine(self, partial, shards, segments, dim, groups, out, seg_len=None, avg=False):
        p = partial.numpy().reshape(shards, segments, dim)
        acc = np.zeros((segments, dim), np.float32)
        for w in range(shards):
            acc = acc + p[w]
        if avg:
            sl = seg_len.numpy()
            scale = np.where(sl != 0, (1.0 / np.maximum(sl, 1)).astype(np.float32), np.float32(1))
            acc = acc * scale[:, None]
        rows = segments // groups
        o = out.numpy()
        for g in range(groups):
            o[:, g * dim:(g + 1) * dim] = acc[g * rows:(g + 1) * rows]
        return out
