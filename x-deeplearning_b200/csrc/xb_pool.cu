// Embedding pooling over variable-length id lists, and the HBM table image.
//
// Three kernels share one geometry: a table row is fetched by LPR lanes with 128-bit loads (lane c
// reads bytes [16c,16c+16) of the row) and accumulated in fp32.
//   pool_queue_kernel  sum / average, one output per feature group, large batches: one sub-team of LPR
//                      lanes per segment, 32 segments per warp handed out as sub-teams finish.
//   pool_fast_kernel   one output per feature group (kAssign included), any batch: teams of TL lanes
//                      per segment, TL/LPR sub-teams that walk the ids s, s+NS, s+2NS..., combined
//                      with a fixed xor butterfly.
//   pool_kernel        several outputs per feature group (the general case), same team layout.
// In every kernel the order in which a segment's rows are added is fixed by the geometry alone, so a
// result does not depend on scheduling. Per id the kernels move 8 B id + 4 B value + one row.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "xb_common.cuh"

namespace xb {

struct PoolItemDev {
  int32_t udf, trunc_dir, trunc_num, assign_stride;
  void* out;
  int64_t stride;
};

struct PoolGroupDev {
  const char* weights;
  const int64_t* slot_keys;
  const int32_t* slot_rows;
  const void* ids;
  const void* values;
  const int32_t* offsets;      // exclusive offsets [batch+1]
  int64_t rows, pitch, slot_mask, batch;
  int64_t warp_begin;          // first warp of this group in the launch
  int32_t dim, tdtype, id_dtype, out_dtype, n_items, has_table;
  int32_t lpr;                 // lanes per row
  int32_t tl;                  // lanes per segment (team)
  int32_t vhalf;               // per-id weights are fp16
  int32_t segs;                // specialised kernel: rounds of segments per warp
  PoolItemDev items[XB_MAX_POOL_ITEMS];
};

struct PoolParams {
  int32_t n_groups;
  int64_t total_warps;
  PoolGroupDev g[XB_MAX_POOL_GROUPS];
};

struct ScanParams {
  int32_t n;
  const int32_t* counts[XB_MAX_POOL_GROUPS];
  int32_t* offsets[XB_MAX_POOL_GROUPS];
  int64_t batch[XB_MAX_POOL_GROUPS];
  // multi-CTA form: chunks of SCAN_THREADS * SCAN_ITEMS counts, numbered across the groups
  int32_t* chunk_sums[XB_MAX_POOL_GROUPS];
  int32_t chunk_begin[XB_MAX_POOL_GROUPS + 1];
};

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33; return x;
}

// counts -> exclusive offsets, one CTA per group: 1024 threads x 8 counts per pass (8192 per pass).
constexpr int SCAN_THREADS = 1024, SCAN_ITEMS = 8;
__global__ void __launch_bounds__(SCAN_THREADS) scan_counts_kernel(const __grid_constant__ ScanParams p) {
  const int g = blockIdx.x;
  const int32_t* __restrict__ counts = p.counts[g];
  int32_t* __restrict__ offsets = p.offsets[g];
  const int64_t batch = p.batch[g];
  __shared__ int32_t warp_sums[SCAN_THREADS / 32];
  __shared__ int32_t carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool vec = (reinterpret_cast<uintptr_t>(counts) & 15) == 0;
  for (int64_t base = 0; base < batch; base += SCAN_THREADS * SCAN_ITEMS) {
    const int64_t i0 = base + (int64_t)threadIdx.x * SCAN_ITEMS;
    int32_t c[SCAN_ITEMS];
    if (vec && i0 + SCAN_ITEMS <= batch) {
      const int4 a = __ldg(reinterpret_cast<const int4*>(counts + i0));
      const int4 b = __ldg(reinterpret_cast<const int4*>(counts + i0) + 1);
      c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < SCAN_ITEMS; ++e) c[e] = (i0 + e < batch) ? counts[i0 + e] : 0;
    }
    int32_t tsum = 0;
#pragma unroll
    for (int e = 0; e < SCAN_ITEMS; ++e) tsum += c[e];
    int32_t incl = tsum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int32_t v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    // the first warp scans the 32 warp totals
    if (warp == 0) {
      int32_t w = warp_sums[lane], wi = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int32_t v = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += v;
      }
      warp_sums[lane] = wi - w;          // exclusive
    }
    __syncthreads();
    const int32_t carry = carry_s;
    int32_t excl = carry + warp_sums[warp] + incl - tsum;
#pragma unroll
    for (int e = 0; e < SCAN_ITEMS; ++e) {
      if (i0 + e < batch) offsets[i0 + e] = excl;
      excl += c[e];
    }
    __syncthreads();
    if (threadIdx.x == SCAN_THREADS - 1) carry_s = excl;      // running total after this pass
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[batch] = carry_s;
}

// Multi-CTA form for long count arrays, two launches: every CTA sums its chunk; then every CTA adds up the
// sums of the chunks before it (same group) and scans its own chunk from that base.
__device__ __forceinline__ int scan_find_group(const ScanParams& p, int chunk) {
  int g = 0;
  while (g + 1 < p.n && p.chunk_begin[g + 1] <= chunk) ++g;
  return g;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_sums_kernel(const __grid_constant__ ScanParams p) {
  const int g = scan_find_group(p, blockIdx.x), lc = blockIdx.x - p.chunk_begin[g];
  const int32_t* __restrict__ counts = p.counts[g];
  const int64_t batch = p.batch[g], i0 = (int64_t)lc * SCAN_THREADS * SCAN_ITEMS + (int64_t)threadIdx.x * SCAN_ITEMS;
  __shared__ int32_t warp_sums[SCAN_THREADS / 32];
  int32_t s = 0;
#pragma unroll
  for (int e = 0; e < SCAN_ITEMS; ++e) s += (i0 + e < batch) ? counts[i0 + e] : 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    int32_t w = warp_sums[threadIdx.x];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) w += __shfl_xor_sync(0xffffffffu, w, off);
    if (threadIdx.x == 0) p.chunk_sums[g][lc] = w;
  }
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_apply_kernel(const __grid_constant__ ScanParams p) {
  const int g = scan_find_group(p, blockIdx.x), lc = blockIdx.x - p.chunk_begin[g];
  const int32_t* __restrict__ counts = p.counts[g];
  int32_t* __restrict__ offsets = p.offsets[g];
  const int64_t batch = p.batch[g];
  __shared__ int32_t warp_sums[SCAN_THREADS / 32];
  __shared__ int32_t base_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // base = sum of the chunk sums before this chunk (integer sums: any order gives the same value)
  int32_t b = 0;
  for (int c = threadIdx.x; c < lc; c += SCAN_THREADS) b += p.chunk_sums[g][c];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) b += __shfl_xor_sync(0xffffffffu, b, off);
  if (lane == 0) warp_sums[warp] = b;
  __syncthreads();
  if (warp == 0) {
    int32_t w = warp_sums[lane];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) w += __shfl_xor_sync(0xffffffffu, w, off);
    if (lane == 0) base_s = w;
  }
  __syncthreads();
  const int32_t base = base_s;
  const int64_t i0 = (int64_t)lc * SCAN_THREADS * SCAN_ITEMS + (int64_t)threadIdx.x * SCAN_ITEMS;
  int32_t c[SCAN_ITEMS];
#pragma unroll
  for (int e = 0; e < SCAN_ITEMS; ++e) c[e] = (i0 + e < batch) ? counts[i0 + e] : 0;
  int32_t tsum = 0;
#pragma unroll
  for (int e = 0; e < SCAN_ITEMS; ++e) tsum += c[e];
  int32_t incl = tsum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int32_t v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  __syncthreads();                       // warp_sums is reused
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t w = warp_sums[lane], wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int32_t v = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += v;
    }
    warp_sums[lane] = wi - w;            // exclusive
  }
  __syncthreads();
  int32_t excl = base + warp_sums[warp] + incl - tsum;
#pragma unroll
  for (int e = 0; e < SCAN_ITEMS; ++e) {
    if (i0 + e < batch) offsets[i0 + e] = excl;
    excl += c[e];
  }
  // the thread that holds the last count of the group also writes the total
  if (i0 < batch && i0 + SCAN_ITEMS >= batch) offsets[batch] = excl;
}

__device__ __forceinline__ int64_t lookup_row(const PoolGroupDev& g, int64_t key) {
  if (g.slot_keys == nullptr) return (key >= 0 && key < g.rows) ? key : -1;
  uint64_t h = mix64((uint64_t)key) & (uint64_t)g.slot_mask;
  // bounded probe: an index built by xb_table_build_index_host is at most half full
  for (int64_t probes = 0; probes <= g.slot_mask; ++probes) {
    int32_t r = __ldg(g.slot_rows + h);
    if (r < 0) return -1;
    if (__ldg(g.slot_keys + h) == key) return r;
    h = (h + 1) & (uint64_t)g.slot_mask;
  }
  return -1;
}

__device__ __forceinline__ void unpack_chunk(const uint4& raw, int tdtype, float (&w)[8]) {
  if (tdtype == XB_F32) {
    w[0] = __uint_as_float(raw.x); w[1] = __uint_as_float(raw.y);
    w[2] = __uint_as_float(raw.z); w[3] = __uint_as_float(raw.w);
    w[4] = w[5] = w[6] = w[7] = 0.f;
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __half22float2(h[e]);
      w[2 * e] = f.x; w[2 * e + 1] = f.y;
    }
  }
}

// Per-load cache behaviour. Table rows are the data worth keeping: they are read with an L2 evict_last
// policy, so the hot rows of a Zipf-distributed id stream stay resident while the streams that are touched
// once (ids, per-id weights, outputs) pass through with streaming loads and stores (evict first).
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ld_row16(const void* ptr, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr), "l"(policy));
  return v;
}

__device__ __forceinline__ uint4 load_row_chunk(const PoolGroupDev& g, int64_t row, int chunk) {
  const uint4* p = reinterpret_cast<const uint4*>(g.weights + row * g.pitch) + chunk;
  return __ldg(p);
}

__device__ __forceinline__ void store_out(void* out, int64_t idx, int out_dtype, float v) {
  if (out_dtype == XB_F32) reinterpret_cast<float*>(out)[idx] = v;
  else reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
}

__global__ void __launch_bounds__(256) pool_kernel(const __grid_constant__ PoolParams p) {
  const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= p.total_warps) return;      // whole warp leaves together
  const int lane = threadIdx.x & 31;
  int gi = 0;
  while (gi + 1 < p.n_groups && p.g[gi + 1].warp_begin <= warp_id) ++gi;
  const PoolGroupDev& g = p.g[gi];

  const int tl = g.tl, lpr = g.lpr;
  const int team = lane / tl, tlane = lane % tl;
  const int sub = tlane / lpr, chunk = tlane % lpr;
  const int ns = tl / lpr;
  const int epc = (g.tdtype == XB_F32) ? 4 : 8;          // elements per 16-byte chunk
  const int col0 = chunk * epc;
  const int64_t seg = (warp_id - g.warp_begin) * (32 / tl) + team;
  const bool active = seg < g.batch;
  const bool loads = active && g.has_table && col0 < g.dim;

  int64_t start = 0, num = 0;
  if (active) {
    start = g.offsets[seg];
    num = (int64_t)g.offsets[seg + 1] - start;
  }

  // kAssign items: clear the item's span first (the reference memsets it in
  // InitProcess), then every fetched row is written straight to its slot.
  bool any_assign = false;
  for (int k = 0; k < g.n_items; ++k) {
    const PoolItemDev& it = g.items[k];
    if (it.udf != XB_UDF_ASSIGN) continue;
    any_assign = true;
    if (active) {
      const int as = it.assign_stride ? it.assign_stride : g.dim;
      const int64_t base = seg * it.stride;
      for (int i = tlane; i < it.trunc_num * g.dim; i += tl) {
        int t = i / g.dim, e = i - t * g.dim;
        store_out(it.out, base + (int64_t)t * as + e, g.out_dtype, 0.f);
      }
    }
  }
  if (any_assign) __syncwarp();

  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;

  if (loads) {
    const bool id64 = g.id_dtype != XB_I32;
    const bool rec = g.id_dtype == XB_REC64;                                // routing records: the row is the low half
    for (int64_t j = sub; j < num; j += 2 * ns) {
      // two ids in flight per sub-team
      const int64_t j1 = j + ns;
      const bool has1 = j1 < num;
      int64_t key0 = id64 ? __ldg(reinterpret_cast<const int64_t*>(g.ids) + start + j)
                          : (int64_t)__ldg(reinterpret_cast<const int32_t*>(g.ids) + start + j);
      int64_t key1 = 0;
      if (has1) key1 = id64 ? __ldg(reinterpret_cast<const int64_t*>(g.ids) + start + j1)
                            : (int64_t)__ldg(reinterpret_cast<const int32_t*>(g.ids) + start + j1);
      if (rec) { key0 &= 0xffffffffll; key1 &= 0xffffffffll; }
      float v0 = 1.f, v1 = 1.f;
      if (g.values) {
        if (g.vhalf) {
          v0 = __half2float(reinterpret_cast<const __half*>(g.values)[start + j]);
          if (has1) v1 = __half2float(reinterpret_cast<const __half*>(g.values)[start + j1]);
        } else {
          v0 = __ldg(reinterpret_cast<const float*>(g.values) + start + j);
          if (has1) v1 = __ldg(reinterpret_cast<const float*>(g.values) + start + j1);
        }
      }
      int64_t r0 = lookup_row(g, key0);
      int64_t r1 = has1 ? lookup_row(g, key1) : -1;
      uint4 raw0 = make_uint4(0, 0, 0, 0), raw1 = make_uint4(0, 0, 0, 0);
      if (r0 >= 0) raw0 = load_row_chunk(g, r0, chunk);
      if (r1 >= 0) raw1 = load_row_chunk(g, r1, chunk);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int64_t r = u ? r1 : r0;
        if (r < 0) continue;                    // missing key contributes nothing
        const int64_t jj = u ? j1 : j;
        const float v = u ? v1 : v0;
        float w[8];
        unpack_chunk(u ? raw1 : raw0, g.tdtype, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = acc[e] + v * w[e];
        for (int k = 0; k < g.n_items; ++k) {
          const PoolItemDev& it = g.items[k];
          if (it.udf != XB_UDF_ASSIGN) continue;
          const int64_t tn = it.trunc_num;
          int64_t slot;
          if (it.trunc_dir == XB_TRUNC_ORDER) {
            if (jj >= tn) continue;
            slot = jj;
          } else {
            if (num - jj > tn) continue;
            slot = tn - (num - jj);
          }
          const int as = it.assign_stride ? it.assign_stride : g.dim;
          const int64_t o = seg * it.stride + slot * as + col0;
          for (int e = 0; e < epc; ++e)
            if (col0 + e < g.dim) store_out(it.out, o + e, g.out_dtype, v * w[e]);
        }
      }
    }
  }

  // fixed-order combine of the sub-team partial sums
  __syncwarp();
  for (int off = lpr; off < tl; off <<= 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
  }

  if (active && sub == 0 && col0 < g.dim) {
    for (int k = 0; k < g.n_items; ++k) {
      const PoolItemDev& it = g.items[k];
      if (it.udf == XB_UDF_ASSIGN) continue;
      float scale = 1.f;
      if (it.udf == XB_UDF_AVG && num != 0) scale = (float)(1.0 / (double)num);
      const int64_t o = seg * it.stride + col0;
      const bool avg = it.udf == XB_UDF_AVG && num != 0;
      float r[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = avg ? acc[e] * scale : acc[e];
      const int nvalid = min(epc, g.dim - col0);
      if (g.out_dtype == XB_F32) {
        float* dst = reinterpret_cast<float*>(it.out) + o;
        if (nvalid == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
          *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
        } else {
          for (int e = 0; e < nvalid; ++e) dst[e] = r[e];
        }
      } else {
        __half* dst = reinterpret_cast<__half*>(it.out) + o;
        if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
          // 32-bit stores of column pairs; an odd tail column goes alone
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            if (e + 1 < nvalid) *reinterpret_cast<__half2*>(dst + e) = __floats2half2_rn(r[e], r[e + 1]);
            else if (e < nvalid) dst[e] = __float2half_rn(r[e]);
          }
        } else {
          for (int e = 0; e < nvalid; ++e) dst[e] = __float2half_rn(r[e]);
        }
      }
    }
  }
}

// Widest aligned store of `nvalid` (<= N) consecutive outputs starting at element index `o`.
template <int N>
__device__ __forceinline__ void store_vec(void* out, int64_t o, bool out16, const float (&r)[N], int nvalid) {
  if (!out16) {
    float* dst = reinterpret_cast<float*>(out) + o;
    if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int e = 0; e < N; e += 4) {
        if (e + 4 <= nvalid) __stcs(reinterpret_cast<float4*>(dst + e), make_float4(r[e], r[e + 1], r[e + 2], r[e + 3]));
        else {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (e + u < nvalid) dst[e + u] = r[e + u];
        }
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e)
        if (e < nvalid) dst[e] = r[e];
    }
  } else {
    __half* dst = reinterpret_cast<__half*>(out) + o;
    const uintptr_t a = reinterpret_cast<uintptr_t>(dst);
    if (N == 8 && nvalid == 8 && (a & 15) == 0) {
      uint4 v;
      __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(r[2 * e], r[2 * e + 1]);
      __stcs(reinterpret_cast<uint4*>(dst), v);
    } else if ((a & 3) == 0) {
#pragma unroll
      for (int e = 0; e < N; e += 2) {
        if (e + 1 < nvalid) *reinterpret_cast<__half2*>(dst + e) = __floats2half2_rn(r[e], r[e + 1]);
        else if (e < nvalid) dst[e] = __float2half_rn(r[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < N; ++e)
        if (e < nvalid) dst[e] = __float2half_rn(r[e]);
    }
  }
}

// Single-item groups (one output per feature group: the usual case), specialised per table dtype
// and lanes per row. Same team / sub-team geometry and the same summation order as pool_kernel
// (sub-team s adds ids s, s+NS, s+2NS... in order, then the xor butterfly), so both kernels give
// identical bits. What differs is the instruction count per id: a team loads TL ids, values and
// row numbers with one coalesced load each (the index lookup runs once per id, not once per
// lane), hands them to the sub-teams by shuffle and keeps up to four 16-byte row loads per lane
// in flight.
template <int TD, int LPR>
__global__ void __launch_bounds__(256, 4) pool_fast_kernel(const __grid_constant__ PoolParams p) {
  constexpr int EPC = TD == XB_F32 ? 4 : 8;          // elements per 16-byte chunk
  constexpr int RB = LPR < 4 ? LPR : 4;              // row loads in flight per lane
  constexpr unsigned FULL = 0xffffffffu;
  const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= p.total_warps) return;              // whole warp leaves together
  const int lane = threadIdx.x & 31;
  int gi = 0;
  while (gi + 1 < p.n_groups && p.g[gi + 1].warp_begin <= warp_id) ++gi;
  const PoolGroupDev& g = p.g[gi];
  const PoolItemDev& it = g.items[0];

  const int tl = g.tl, ns = tl / LPR, spw = 32 / tl, segs = g.segs;
  const int tlane = lane & (tl - 1), team0 = lane - tlane;
  const int sub = tlane / LPR, chunk = tlane & (LPR - 1);
  const int dim = g.dim, col0 = chunk * EPC;
  const bool cvalid = col0 < dim;
  const int nvalid = min(EPC, dim - col0);
  const bool id64 = g.id_dtype != XB_I32, has_table = g.has_table != 0, out16 = g.out_dtype == XB_F16;
  const bool rec = g.id_dtype == XB_REC64;                                  // routing records: the row is the low half
  const int vmode = g.values ? (g.vhalf ? 2 : 1) : 0;
  const bool assign = it.udf == XB_UDF_ASSIGN, avg = it.udf == XB_UDF_AVG;
  const int tn = it.trunc_num, as = it.assign_stride ? it.assign_stride : dim;
  const bool reverse = it.trunc_dir != XB_TRUNC_ORDER;
  const char* wrow = g.weights + chunk * 16;
  const int pitch = (int)g.pitch;                    // a row is at most 256 bytes here: 32 x 32 -> 64-bit multiply
  const uint64_t keep = l2_policy_keep();
  const int64_t batch = g.batch;
  // this warp walks `segs` consecutive rounds of `spw` segments; the offsets of round i+2 and the ids of
  // round i+1 are fetched while the rows of round i are in flight
  const int64_t seg_first = (warp_id - g.warp_begin) * segs * spw + lane / tl;

  auto load_span = [&](int i, int& st, int& nm) {
    const int64_t sg = seg_first + (int64_t)i * spw;
    st = 0; nm = 0;
    if (i < segs && sg < batch) {
      st = __ldg(g.offsets + sg);
      nm = __ldg(g.offsets + sg + 1) - st;
    }
  };
  // one id, value and table row number per lane: position base + tlane of the segment
  auto load_ids = [&](int st, int nm, int base, int& row, float& v) {
    const int idx = base + tlane;
    row = -1; v = 1.f;
    if (idx < nm) {
      const int64_t at = (int64_t)st + idx;
      int64_t key = id64 ? (int64_t)__ldcs(reinterpret_cast<const long long*>(g.ids) + at)
                         : (int64_t)__ldcs(reinterpret_cast<const int32_t*>(g.ids) + at);
      if (rec) key &= 0xffffffffll;
      if (has_table) row = (int)lookup_row(g, key);
      if (vmode == 1) v = __ldcs(reinterpret_cast<const float*>(g.values) + at);
      else if (vmode == 2) v = __half2float(reinterpret_cast<const __half*>(g.values)[at]);
    }
  };

  int st0, nm0, st1, nm1, st2, nm2, row, row_next;
  float v, v_next;
  load_span(0, st0, nm0);
  load_span(1, st1, nm1);
  load_ids(st0, nm0, 0, row, v);
  for (int i = 0; i < segs; ++i) {
    const int64_t seg = seg_first + (int64_t)i * spw;
    if (seg - lane / tl >= batch) break;               // uniform: this round starts past the last segment
    load_span(i + 2, st2, nm2);
    load_ids(st1, nm1, 0, row_next, v_next);
    const bool active = seg < batch;
    const int start = st0, num = nm0;
    const int64_t obase = seg * it.stride + col0;
    float acc[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) acc[e] = 0.f;

    for (int base = 0; __any_sync(FULL, base < num); base += tl) {
      if (base > 0) load_ids(start, num, base, row, v);
#pragma unroll
      for (int r0 = 0; r0 < LPR; r0 += RB) {
        if (r0 > 0 && !__any_sync(FULL, base + r0 * ns < num)) break;      // no team has ids left in this batch
        int rr[RB];
        float vv[RB];
        uint4 raw[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
          const int src = team0 + (r0 + u) * ns + sub;
          rr[u] = __shfl_sync(FULL, row, src);
          vv[u] = __shfl_sync(FULL, v, src);
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
          raw[u] = make_uint4(0, 0, 0, 0);
          if (rr[u] >= 0 && cvalid) raw[u] = ld_row16(wrow + (int64_t)rr[u] * pitch, keep);
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
          float w[8];
          unpack_chunk(raw[u], TD, w);
          if (!assign) {
            if (rr[u] >= 0) {                       // a missing key contributes nothing
#pragma unroll
              for (int e = 0; e < EPC; ++e) acc[e] = acc[e] + vv[u] * w[e];
            }
          } else {
            // kAssign: the id at position jj of the segment owns one output slot; a missing key leaves zeros
            const int jj = base + (r0 + u) * ns + sub;
            if (jj < num && cvalid) {
              int slot = -1;
              if (!reverse) { if (jj < tn) slot = jj; }
              else if (num - jj <= tn) slot = tn - (num - jj);
              if (slot >= 0) {
                float o[EPC];
#pragma unroll
                for (int e = 0; e < EPC; ++e) o[e] = rr[u] >= 0 ? vv[u] * w[e] : 0.f;
                store_vec<EPC>(it.out, obase + (int64_t)slot * as, out16, o, nvalid);
              }
            }
          }
        }
      }
    }

    if (assign) {
      // slots no id maps to are cleared (the reference memsets the whole span first)
      if (active) {
        const int used = min(num, tn), nz = tn - used, z0 = reverse ? 0 : used;
        for (int k = tlane; k < nz * dim; k += tl) {
          const int t = k / dim, e = k - t * dim;
          store_out(it.out, seg * it.stride + (int64_t)(z0 + t) * as + e, g.out_dtype, 0.f);
        }
      }
    } else {
      // fixed-order combine of the sub-team partial sums
      for (int off = LPR; off < tl; off <<= 1) {
#pragma unroll
        for (int e = 0; e < EPC; ++e) acc[e] += __shfl_xor_sync(FULL, acc[e], off);
      }
      if (active && sub == 0 && cvalid) {
        if (avg && num != 0) {
          const float scale = (float)(1.0 / (double)num);
#pragma unroll
          for (int e = 0; e < EPC; ++e) acc[e] = acc[e] * scale;
        }
        store_vec<EPC>(it.out, obase, out16, acc, nvalid);
      }
    }
    st0 = st1; nm0 = nm1; st1 = st2; nm1 = nm2; row = row_next; v = v_next;
  }
}

// Sum / average pooling of very short segments (fewer than three ids on average, large calls): LPR lanes per
// segment, 32 / LPR segments per warp, four row loads in flight per lane, nothing else - no shuffles, no queue,
// no sub-teams. The other kernels spend about 1500 warp instructions per round whatever the segments hold; with
// one or two ids per segment that, not memory, is what a launch costs (an owner rank of an 8-way sharded table
// pools 2.6 M segments of 1.9 ids). A segment's rows are added in id order, as everywhere.
template <int TD, int LPR, bool REC>
__global__ void __launch_bounds__(256) pool_short_kernel(const __grid_constant__ PoolParams p) {
  constexpr int EPC = TD == XB_F32 ? 4 : 8;          // elements per 16-byte chunk
  constexpr int SPW = 32 / LPR;                      // segments per warp and round
  constexpr int U = 4;                               // ids of a segment fetched together
  const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= p.total_warps) return;
  const int lane = threadIdx.x & 31;
  int gi = 0;
  while (gi + 1 < p.n_groups && p.g[gi + 1].warp_begin <= warp_id) ++gi;
  const PoolGroupDev& g = p.g[gi];
  const PoolItemDev& it = g.items[0];
  const int chunk = lane & (LPR - 1);
  const int rounds = g.segs;                         // consecutive rounds of SPW segments this warp walks
  const int64_t seg0 = (warp_id - g.warp_begin) * rounds * SPW + lane / LPR;
  const int64_t batch = g.batch;
  const int dim = g.dim, col0 = chunk * EPC;
  const bool cvalid = col0 < dim;
  const int nvalid = min(EPC, dim - col0);
  const bool id64 = REC || g.id_dtype == XB_I64, has_table = g.has_table != 0, out16 = g.out_dtype == XB_F16;
  const int vmode = g.values ? (g.vhalf ? 2 : 1) : 0;
  const bool avg = it.udf == XB_UDF_AVG;
  const char* wrow = g.weights + chunk * 16;
  const int pitch = (int)g.pitch;
  const uint64_t keep = l2_policy_keep();

  // the offsets of round i+2 and the ids of round i+1 are requested while the rows of round i are in flight, so
  // a round exposes one fetch latency (its rows), not three
  auto load_span = [&](int i, int& st, int& nm) {
    const int64_t sg = seg0 + (int64_t)i * SPW;
    st = 0; nm = 0;
    if (i < rounds && sg < batch) {
      st = __ldg(g.offsets + sg);
      nm = __ldg(g.offsets + sg + 1) - st;
    }
  };
  auto load_ids = [&](int st, int nm, int j, int (&rr)[U], float (&vv)[U]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      rr[u] = -1; vv[u] = 1.f;
      if (j + u < nm) {
        const int64_t at = (int64_t)st + j + u;
        int64_t key = id64 ? (int64_t)__ldcs(reinterpret_cast<const long long*>(g.ids) + at)
                           : (int64_t)__ldcs(reinterpret_cast<const int32_t*>(g.ids) + at);
        if (REC) key &= 0xffffffffll;                           // the row is the low half of a record
        if (has_table) rr[u] = (int)lookup_row(g, key);
        if (vmode == 1) vv[u] = __ldcs(reinterpret_cast<const float*>(g.values) + at);
        else if (vmode == 2) vv[u] = __half2float(reinterpret_cast<const __half*>(g.values)[at]);
      }
    }
  };
  int st0, nm0, st1, nm1, st2, nm2;
  int rr[U], rr_next[U];
  float vv[U], vv_next[U];
  load_span(0, st0, nm0);
  load_span(1, st1, nm1);
  load_ids(st0, nm0, 0, rr, vv);
  for (int i = 0; i < rounds; ++i) {
    const int64_t seg = seg0 + (int64_t)i * SPW;
    load_span(i + 2, st2, nm2);
    load_ids(st1, nm1, 0, rr_next, vv_next);
    float acc[EPC];
#pragma unroll
    for (int e = 0; e < EPC; ++e) acc[e] = 0.f;
    for (int j = 0; j < nm0; j += U) {
      if (j > 0) load_ids(st0, nm0, j, rr, vv);                 // a segment longer than U ids: the rare case here
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        raw[u] = make_uint4(0, 0, 0, 0);
        if (rr[u] >= 0 && cvalid) raw[u] = ld_row16(wrow + (int64_t)rr[u] * pitch, keep);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (rr[u] >= 0) {                                       // a missing key contributes nothing
          float w[8];
          unpack_chunk(raw[u], TD, w);
#pragma unroll
          for (int e = 0; e < EPC; ++e) acc[e] = acc[e] + vv[u] * w[e];
        }
      }
    }
    if (seg < batch && cvalid) {
      if (avg && nm0 != 0) {
        const float scale = (float)(1.0 / (double)nm0);
#pragma unroll
        for (int e = 0; e < EPC; ++e) acc[e] = acc[e] * scale;
      }
      store_vec<EPC>(it.out, seg * it.stride + col0, out16, acc, nvalid);
    }
    st0 = st1; nm0 = nm1; st1 = st2; nm1 = nm2;
#pragma unroll
    for (int u = 0; u < U; ++u) { rr[u] = rr_next[u]; vv[u] = vv_next[u]; }
  }
}

// Sum / average pooling with one sub-team (LPR lanes) per segment and a per-warp segment queue: a warp
// owns 32 consecutive segments, its 32/LPR sub-teams each take the next unclaimed one as soon as they
// finish theirs, so lanes stay busy whatever the spread of segment lengths. A sub-team adds the ids of its
// segment strictly in order (no cross-lane combine). The ids of the batch after the current one are
// requested before the rows of the current one, so both latencies overlap.
// REC: the id lists are routing records (XB_REC64); a template parameter so that the usual instantiation carries
// nothing for it (a run-time test here cost 15 % on tables that do not fit L2)
template <int TD, int LPR, bool REC>
__global__ void __launch_bounds__(256, 4) pool_queue_kernel(const __grid_constant__ PoolParams p) {
  constexpr int EPC = TD == XB_F32 ? 4 : 8;
  constexpr unsigned FULL = 0xffffffffu;
  constexpr int NT = 32 / LPR;                       // sub-teams per warp
  const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= p.total_warps) return;
  const int lane = threadIdx.x & 31;
  int gi = 0;
  while (gi + 1 < p.n_groups && p.g[gi + 1].warp_begin <= warp_id) ++gi;
  const PoolGroupDev& g = p.g[gi];
  const PoolItemDev& it = g.items[0];

  const int tlane = lane & (LPR - 1), team0 = lane - tlane, team = lane / LPR;
  const int dim = g.dim, col0 = tlane * EPC;
  const bool cvalid = col0 < dim;
  const int nvalid = min(EPC, dim - col0);
  const bool id64 = REC || g.id_dtype == XB_I64, has_table = g.has_table != 0, out16 = g.out_dtype == XB_F16;
  const int vmode = g.values ? (g.vhalf ? 2 : 1) : 0;
  const bool avg = it.udf == XB_UDF_AVG;
  const char* wrow = g.weights + tlane * 16;
  const int pitch = (int)g.pitch;
  const uint64_t keep = l2_policy_keep();
  const int64_t s0 = (warp_id - g.warp_begin) * 32;
  const int nseg = (int)min((int64_t)32, g.batch - s0);

  // lane l keeps the span of segment s0 + l
  int my_start = 0, my_num = 0;
  if (lane < nseg) {
    my_start = __ldg(g.offsets + s0 + lane);
    my_num = __ldg(g.offsets + s0 + lane + 1) - my_start;
  }
  auto load_ids = [&](int st, int nm, int pos, int& row, float& v) {
    const int idx = pos + tlane;
    row = -1; v = 1.f;
    if (idx < nm) {
      const int64_t at = (int64_t)st + idx;
      int64_t key = id64 ? (int64_t)__ldcs(reinterpret_cast<const long long*>(g.ids) + at)
                         : (int64_t)__ldcs(reinterpret_cast<const int32_t*>(g.ids) + at);
      if (REC) key &= 0xffffffffll;                           // the row is the low half of a record
      if (has_table) row = (int)lookup_row(g, key);
      if (vmode == 1) v = __ldcs(reinterpret_cast<const float*>(g.values) + at);
      else if (vmode == 2) v = __half2float(reinterpret_cast<const __half*>(g.values)[at]);
    }
  };

  int m = team, next = NT;                           // my segment (relative), first unclaimed one
  int start = __shfl_sync(FULL, my_start, m & 31), num = __shfl_sync(FULL, my_num, m & 31);
  if (m >= nseg) num = 0;
  int pos = 0, row;
  float v;
  load_ids(start, num, 0, row, v);
  float acc[EPC];
#pragma unroll
  for (int e = 0; e < EPC; ++e) acc[e] = 0.f;

  while (__any_sync(FULL, m < nseg)) {
    // where this sub-team goes after the current batch: on in its segment, or to the next unclaimed one
    const bool live = m < nseg;
    const bool finishing = live && pos + LPR >= num;
    const unsigned fmask = __ballot_sync(FULL, finishing && tlane == 0);
    int m2 = m, pos2 = pos + LPR, start2 = start, num2 = num;
    if (fmask) {
      const int cand = next + __popc(fmask & ((1u << team0) - 1u));
      const int cs = __shfl_sync(FULL, my_start, cand & 31), cn = __shfl_sync(FULL, my_num, cand & 31);
      if (finishing) {
        m2 = cand; pos2 = 0; start2 = cs;
        num2 = cand < nseg ? cn : 0;
      }
      next += __popc(fmask);
    }
    int row2;
    float v2;
    load_ids(start2, m2 < nseg ? num2 : 0, pos2, row2, v2);

    // rows of the current batch: id r of the batch sits in lane team0 + r
    int rr[LPR];
    float vv[LPR];
#pragma unroll
    for (int r = 0; r < LPR; ++r) {
      rr[r] = __shfl_sync(FULL, row, team0 + r);
      vv[r] = __shfl_sync(FULL, v, team0 + r);
    }
#pragma unroll
    for (int r0 = 0; r0 < LPR; r0 += 4) {
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        raw[u] = make_uint4(0, 0, 0, 0);
        if (r0 + u < LPR && rr[r0 + u] >= 0 && cvalid)
          raw[u] = ld_row16(wrow + (int64_t)rr[r0 + u] * pitch, keep);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r0 + u < LPR && rr[r0 + u] >= 0) {             // a missing key contributes nothing
          float w[8];
          unpack_chunk(raw[u], TD, w);
#pragma unroll
          for (int e = 0; e < EPC; ++e) acc[e] = acc[e] + vv[r0 + u] * w[e];
        }
      }
    }
    if (finishing) {
      if (cvalid) {
        if (avg && num != 0) {
          const float scale = (float)(1.0 / (double)num);
#pragma unroll
          for (int e = 0; e < EPC; ++e) acc[e] = acc[e] * scale;
        }
        store_vec<EPC>(it.out, (s0 + m) * it.stride + col0, out16, acc, nvalid);
      }
#pragma unroll
      for (int e = 0; e < EPC; ++e) acc[e] = 0.f;
    }
    m = m2; pos = pos2; start = start2; num = num2; row = row2; v = v2;
  }
}

template <int TD, bool REC>
static int launch_pool_queue(const PoolParams& p, int lpr, unsigned blocks, cudaStream_t stream) {
  switch (lpr) {
    case 1: case 2: pool_queue_kernel<TD, 2, REC><<<blocks, 256, 0, stream>>>(p); break;
    case 4: pool_queue_kernel<TD, 4, REC><<<blocks, 256, 0, stream>>>(p); break;
    case 8: pool_queue_kernel<TD, 8, REC><<<blocks, 256, 0, stream>>>(p); break;
    default: pool_queue_kernel<TD, 16, REC><<<blocks, 256, 0, stream>>>(p); break;
  }
  return check_launch("pool_queue_kernel");
}

template <int TD>
static int launch_pool_fast(const PoolParams& p, int lpr, unsigned blocks, cudaStream_t stream) {
  switch (lpr) {
    case 1: case 2: pool_fast_kernel<TD, 2><<<blocks, 256, 0, stream>>>(p); break;
    case 4: pool_fast_kernel<TD, 4><<<blocks, 256, 0, stream>>>(p); break;
    case 8: pool_fast_kernel<TD, 8><<<blocks, 256, 0, stream>>>(p); break;
    default: pool_fast_kernel<TD, 16><<<blocks, 256, 0, stream>>>(p); break;
  }
  return check_launch("pool_fast_kernel");
}

template <int TD, bool REC>
static int launch_pool_short(const PoolParams& p, int lpr, unsigned blocks, cudaStream_t stream) {
  switch (lpr) {
    case 1: case 2: pool_short_kernel<TD, 2, REC><<<blocks, 256, 0, stream>>>(p); break;
    case 4: pool_short_kernel<TD, 4, REC><<<blocks, 256, 0, stream>>>(p); break;
    case 8: pool_short_kernel<TD, 8, REC><<<blocks, 256, 0, stream>>>(p); break;
    default: pool_short_kernel<TD, 16, REC><<<blocks, 256, 0, stream>>>(p); break;
  }
  return check_launch("pool_short_kernel");
}

static int next_pow2(int v) { int p = 1; while (p < v) p <<= 1; return p; }

}  // namespace xb

using namespace xb;

extern "C" int64_t xb_table_row_pitch(int32_t dim, int32_t dtype) {
  size_t es = dtype_size(dtype);
  if (es == 0 || dim <= 0) return 0;
  return (int64_t)(((size_t)dim * es + 15) / 16 * 16);
}

extern "C" int xb_table_build_index_host(const int64_t* keys, int64_t rows, int64_t slots,
                                         int64_t* slot_keys, int32_t* slot_rows) {
  XB_REQUIRE(keys && slot_keys && slot_rows, XB_ERR_ARG, "xb_table_build_index_host: null pointer");
  XB_REQUIRE(slots >= 2 * rows && (slots & (slots - 1)) == 0, XB_ERR_ARG,
             "xb_table_build_index_host: slots=%lld must be a power of two >= 2*rows", (long long)slots);
  XB_REQUIRE(rows < (int64_t)1 << 31, XB_ERR_LIMIT, "xb_table_build_index_host: rows beyond int32");
  for (int64_t i = 0; i < slots; ++i) { slot_rows[i] = -1; slot_keys[i] = 0; }
  const uint64_t mask = (uint64_t)slots - 1;
  for (int64_t r = 0; r < rows; ++r) {
    uint64_t x = (uint64_t)keys[r];
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
    uint64_t h = x & mask;
    while (slot_rows[h] != -1 && slot_keys[h] != keys[r]) h = (h + 1) & mask;
    if (slot_rows[h] == -1) { slot_keys[h] = keys[r]; slot_rows[h] = (int32_t)r; }
  }
  return 0;
}

extern "C" int xb_table_create(xb_table_desc** out, int64_t rows, int32_t dim, int32_t dtype,
                               const float* w, const int64_t* keys) {
  XB_REQUIRE(out && w && rows > 0 && dim > 0, XB_ERR_ARG, "xb_table_create: bad arguments");
  XB_REQUIRE(dtype == XB_F32 || dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_table_create: dtype %d", dtype);
  const int64_t pitch = xb_table_row_pitch(dim, dtype);
  xb_table_desc* t = (xb_table_desc*)calloc(1, sizeof(xb_table_desc));
  t->rows = rows; t->dim = dim; t->dtype = dtype; t->row_pitch_bytes = pitch;
  void* dw = nullptr;
  cudaError_t e = cudaMalloc(&dw, (size_t)rows * pitch);
  if (e != cudaSuccess) { free(t); return fail(XB_ERR_CUDA, "xb_table_create: cudaMalloc %s", cudaGetErrorString(e)); }
  // stage in bounded host chunks so a multi-GB table never needs a second full copy
  const int64_t chunk_rows = std::max<int64_t>(1, (64 << 20) / pitch);
  std::vector<char> stage((size_t)chunk_rows * pitch);
  for (int64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
    const int64_t n = std::min(chunk_rows, rows - r0);
    memset(stage.data(), 0, (size_t)n * pitch);
    for (int64_t r = 0; r < n; ++r) {
      const float* src = w + (r0 + r) * dim;
      if (dtype == XB_F32) memcpy(stage.data() + r * pitch, src, sizeof(float) * dim);
      else {
        __half* d = reinterpret_cast<__half*>(stage.data() + r * pitch);
        for (int c = 0; c < dim; ++c) d[c] = __float2half_rn(src[c]);
      }
    }
    e = cudaMemcpy((char*)dw + r0 * pitch, stage.data(), (size_t)n * pitch, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(dw); free(t); return fail(XB_ERR_CUDA, "xb_table_create: copy %s", cudaGetErrorString(e)); }
  }
  t->weights = dw;
  if (keys) {
    int64_t slots = 16;
    while (slots < 2 * rows) slots <<= 1;
    std::vector<int64_t> sk((size_t)slots);
    std::vector<int32_t> sr((size_t)slots);
    int rc = xb_table_build_index_host(keys, rows, slots, sk.data(), sr.data());
    if (rc) { cudaFree(dw); free(t); return rc; }
    void *dk = nullptr, *dr = nullptr;
    if (cudaMalloc(&dk, slots * 8) != cudaSuccess || cudaMalloc(&dr, slots * 4) != cudaSuccess ||
        cudaMemcpy(dk, sk.data(), slots * 8, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(dr, sr.data(), slots * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
      cudaFree(dw); if (dk) cudaFree(dk); if (dr) cudaFree(dr); free(t);
      return fail(XB_ERR_CUDA, "xb_table_create: index upload failed");
    }
    t->slot_keys = (const int64_t*)dk; t->slot_rows = (const int32_t*)dr; t->slots = slots;
  }
  *out = t;
  return 0;
}

extern "C" int xb_table_clone(xb_table_desc** out, const xb_table_desc* src, int32_t src_device) {
  XB_REQUIRE(out && src && src->weights && src->rows > 0, XB_ERR_ARG, "xb_table_clone: bad arguments");
  int dev = 0;
  XB_CUDA(cudaGetDevice(&dev));
  xb_table_desc* t = (xb_table_desc*)calloc(1, sizeof(xb_table_desc));
  *t = *src;
  t->weights = nullptr; t->slot_keys = nullptr; t->slot_rows = nullptr;
  void *dw = nullptr, *dk = nullptr, *dr = nullptr;
  const size_t wbytes = (size_t)src->rows * src->row_pitch_bytes;
  bool ok = cudaMalloc(&dw, wbytes) == cudaSuccess &&
            cudaMemcpyPeer(dw, dev, src->weights, src_device, wbytes) == cudaSuccess;
  if (ok && src->slot_keys) {
    ok = cudaMalloc(&dk, (size_t)src->slots * 8) == cudaSuccess && cudaMalloc(&dr, (size_t)src->slots * 4) == cudaSuccess &&
         cudaMemcpyPeer(dk, dev, src->slot_keys, src_device, (size_t)src->slots * 8) == cudaSuccess &&
         cudaMemcpyPeer(dr, dev, src->slot_rows, src_device, (size_t)src->slots * 4) == cudaSuccess;
  }
  if (ok) ok = cudaDeviceSynchronize() == cudaSuccess;
  if (!ok) {
    const cudaError_t e = cudaGetLastError();
    if (dw) cudaFree(dw);
    if (dk) cudaFree(dk);
    if (dr) cudaFree(dr);
    free(t);
    return fail(XB_ERR_CUDA, "xb_table_clone: %s", cudaGetErrorString(e));
  }
  t->weights = dw; t->slot_keys = (const int64_t*)dk; t->slot_rows = (const int32_t*)dr;
  *out = t;
  return 0;
}

extern "C" void xb_table_destroy(xb_table_desc* t) {
  if (!t) return;
  if (t->weights) cudaFree((void*)t->weights);
  if (t->slot_keys) cudaFree((void*)t->slot_keys);
  if (t->slot_rows) cudaFree((void*)t->slot_rows);
  free(t);
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
static size_t scan_chunks(int64_t batch) {
  return (size_t)((batch + SCAN_THREADS * SCAN_ITEMS - 1) / (SCAN_THREADS * SCAN_ITEMS));
}

extern "C" size_t xb_embedding_pool_scratch_bytes(const xb_pool_group* groups, int32_t n_groups) {
  size_t total = 0;
  for (int i = 0; i < n_groups; ++i)
    if (!groups[i].segments_are_offsets)
      total += align256(((size_t)groups[i].batch + 1) * 4) + align256(scan_chunks(groups[i].batch) * 4);
  return total;
}

extern "C" int xb_embedding_pool(const xb_pool_group* groups, int32_t n_groups, void* scratch,
                                 size_t scratch_bytes, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(groups && n_groups > 0, XB_ERR_ARG, "xb_embedding_pool: no groups");
  XB_REQUIRE(n_groups <= XB_MAX_POOL_GROUPS, XB_ERR_LIMIT,
             "xb_embedding_pool: %d groups in one call, at most %d", n_groups, XB_MAX_POOL_GROUPS);
  XB_REQUIRE(xb_embedding_pool_scratch_bytes(groups, n_groups) <= scratch_bytes, XB_ERR_SCRATCH,
             "xb_embedding_pool: scratch %zu bytes, need %zu", scratch_bytes,
             xb_embedding_pool_scratch_bytes(groups, n_groups));
  // p: groups for the general kernel; fp[b]: single-item groups for the specialised kernel, one launch
  // per (table dtype, lanes per row) bucket
  constexpr int kBuckets = 8;
  static thread_local PoolParams p;
  static thread_local PoolParams fp[kBuckets];
  static thread_local PoolParams qp[kBuckets];       // segment-queue kernel (sum / average, large batches)
  static thread_local PoolParams hp[kBuckets];       // short-segment kernel (sum / average, fewer than 3 ids a segment)
  static thread_local ScanParams sp;
  p.n_groups = 0;
  p.total_warps = 0;
  for (int b = 0; b < kBuckets; ++b) {
    fp[b].n_groups = 0; fp[b].total_warps = 0; qp[b].n_groups = 0; qp[b].total_warps = 0; hp[b].n_groups = 0; hp[b].total_warps = 0;
  }
  sp.n = 0;
  sp.chunk_begin[0] = 0;
  size_t soff = 0;
  // how much parallelism the whole call offers: the groups of one call share its launches, so the choice between
  // wider teams (more warps, for small calls) and one sub-team per segment (fewest instructions per id, for
  // large ones) looks at all single-output groups together
  int64_t call_segments = 0;
  // the short-segment kernel serves a call only as a whole (a call keeps its number of launches): every group must
  // be a single sum / average output with fewer than three ids per segment on average
  bool all_short = true;
  for (int i = 0; i < n_groups; ++i) {
    if (groups[i].n_items == 1 && groups[i].batch > 0) call_segments += groups[i].batch;
    if (groups[i].batch > 0 &&
        (groups[i].n_items != 1 || groups[i].items[0].udf == XB_UDF_ASSIGN || (double)groups[i].n_ids >= 3.0 * (double)groups[i].batch))
      all_short = false;
  }
  all_short = all_short && (call_segments + 31) / 32 >= (int64_t)sm_count() * 8;
  for (int i = 0; i < n_groups; ++i) {
    const xb_pool_group& h = groups[i];
    XB_REQUIRE(h.batch >= 0 && h.n_ids >= 0, XB_ERR_ARG, "xb_embedding_pool: group %d negative size", i);
    if (h.batch == 0) continue;                // empty group: nothing to write
    XB_REQUIRE(h.n_items >= 1 && h.n_items <= XB_MAX_POOL_ITEMS, XB_ERR_ARG,
               "xb_embedding_pool: group %d has %d items (1..%d)", i, h.n_items, XB_MAX_POOL_ITEMS);
    XB_REQUIRE(h.segments, XB_ERR_ARG, "xb_embedding_pool: group %d without segments", i);
    XB_REQUIRE(h.n_ids == 0 || h.ids, XB_ERR_ARG, "xb_embedding_pool: group %d without ids", i);
    XB_REQUIRE(h.id_dtype == XB_I64 || h.id_dtype == XB_I32 || h.id_dtype == XB_REC64, XB_ERR_UNSUPPORTED,
               "xb_embedding_pool: group %d id dtype %d (int64, int32 or routing records)", i, h.id_dtype);
    XB_REQUIRE(h.out_dtype == XB_F32 || h.out_dtype == XB_F16, XB_ERR_UNSUPPORTED,
               "xb_embedding_pool: group %d output dtype %d", i, h.out_dtype);
    XB_REQUIRE(h.batch < ((int64_t)1 << 31) && h.n_ids < ((int64_t)1 << 31), XB_ERR_LIMIT,
               "xb_embedding_pool: group %d beyond int32 offsets", i);
    PoolGroupDev d;
    memset(&d, 0, sizeof(d));
    d.has_table = h.table != nullptr;
    XB_REQUIRE(h.dim >= 1 && h.dim <= 256, XB_ERR_LIMIT, "xb_embedding_pool: group %d dim %d (1..256)", i, h.dim);
    const int dim = h.dim;
    if (h.table) {
      const xb_table_desc& t = *h.table;
      XB_REQUIRE(t.dtype == XB_F32 || t.dtype == XB_F16, XB_ERR_UNSUPPORTED, "table dtype %d", t.dtype);
      XB_REQUIRE(t.dim == dim, XB_ERR_ARG, "xb_embedding_pool: group %d dim %d, table dim %d", i, dim, t.dim);
      XB_REQUIRE(t.row_pitch_bytes % 16 == 0 && t.row_pitch_bytes >= (int64_t)(t.dim * dtype_size(t.dtype)),
                 XB_ERR_ARG, "xb_embedding_pool: table pitch %lld not a multiple of 16 covering dim %d",
                 (long long)t.row_pitch_bytes, t.dim);
      XB_REQUIRE(((uintptr_t)t.weights & 15) == 0, XB_ERR_ARG, "xb_embedding_pool: table not 16-byte aligned");
      XB_REQUIRE(t.slot_keys == nullptr || (t.slots > 0 && (t.slots & (t.slots - 1)) == 0), XB_ERR_ARG,
                 "xb_embedding_pool: index slots must be a power of two");
      d.weights = (const char*)t.weights; d.rows = t.rows; d.pitch = t.row_pitch_bytes;
      d.slot_keys = t.slot_keys; d.slot_rows = t.slot_rows; d.slot_mask = t.slots - 1;
      d.tdtype = t.dtype;
    } else {
      d.tdtype = XB_F16;   // only fixes the lane geometry: nothing is fetched for a missing table
    }
    d.dim = dim;
    const int epc = d.tdtype == XB_F32 ? 4 : 8;
    d.lpr = next_pow2((dim + epc - 1) / epc);
    if (d.lpr > 32) return fail(XB_ERR_LIMIT, "xb_embedding_pool: row too wide");
    const bool fast = h.n_items == 1 && d.lpr <= 16;
    if (fast && d.lpr < 2) d.lpr = 2;
    const double avg = (double)h.n_ids / (double)h.batch;
    int ns = 1;
    if (fast) {
      // one sub-team per segment gives the fewest instructions per id (no cross-lane combine, whole rows
      // per lane group); teams grow while the launch would otherwise leave SMs without warps, or while a
      // segment is so long that one sub-team would walk it in more than a dozen dependent batches of ids
      // (a 100-step behaviour list on 4 lanes is 25 id-load -> row-load round trips in a row; on a whole warp, 4)
      const int64_t want_warps = (int64_t)sm_count() * 32;
      while (ns < 32 / d.lpr && ns < avg &&
             (call_segments * (int64_t)(d.lpr * ns) / 32 < want_warps || (avg >= 48.0 && avg > 12.0 * ns)))
        ns <<= 1;
    } else {
      while (ns < 32 / d.lpr && ns < avg) ns <<= 1;
    }
    d.tl = d.lpr * ns;
    XB_REQUIRE(h.values_dtype == 0 || h.values_dtype == XB_F32 || h.values_dtype == XB_F16, XB_ERR_UNSUPPORTED,
               "xb_embedding_pool: group %d values dtype %d", i, h.values_dtype);
    d.ids = h.ids; d.values = h.values; d.batch = h.batch; d.vhalf = h.values_dtype == XB_F16;
    d.id_dtype = h.id_dtype; d.out_dtype = h.out_dtype; d.n_items = h.n_items;
    for (int k = 0; k < h.n_items; ++k) {
      const xb_pool_item& it = h.items[k];
      XB_REQUIRE(it.out, XB_ERR_ARG, "xb_embedding_pool: group %d item %d without output", i, k);
      XB_REQUIRE(it.udf >= XB_UDF_SUM && it.udf <= XB_UDF_ASSIGN, XB_ERR_UNSUPPORTED,
                 "Unsupported udf type: %d", it.udf);
      XB_REQUIRE(it.udf != XB_UDF_ASSIGN || it.trunc_num > 0, XB_ERR_ARG,
                 "xb_embedding_pool: kAssign needs trunc_num > 0");
      d.items[k].udf = it.udf; d.items[k].trunc_dir = it.trunc_dir; d.items[k].trunc_num = it.trunc_num;
      d.items[k].assign_stride = it.udf == XB_UDF_ASSIGN ? it.assign_stride : 0;
      d.items[k].out = it.out; d.items[k].stride = it.stride;
    }
    if (h.segments_are_offsets) {
      d.offsets = h.segments;
    } else {
      int32_t* off = reinterpret_cast<int32_t*>((char*)scratch + soff);
      soff += align256(((size_t)h.batch + 1) * 4);
      sp.chunk_sums[sp.n] = reinterpret_cast<int32_t*>((char*)scratch + soff);
      soff += align256(scan_chunks(h.batch) * 4);
      sp.chunk_begin[sp.n + 1] = sp.chunk_begin[sp.n] + (int32_t)scan_chunks(h.batch);
      sp.counts[sp.n] = h.segments; sp.offsets[sp.n] = off; sp.batch[sp.n] = h.batch; ++sp.n;
      d.offsets = off;
    }
    int lg = 0;
    while ((2 << lg) < d.lpr) ++lg;                 // lanes per row 2, 4, 8, 16 -> 0..3
    const int bucket = (d.tdtype == XB_F32 ? 0 : 4) + lg;
    // sum / average groups with plenty of segments go to the segment-queue kernel: 32 segments per warp
    const bool queue = fast && d.tl == d.lpr && h.items[0].udf != XB_UDF_ASSIGN && avg >= 3.0 &&
                       (call_segments + 31) / 32 >= (int64_t)sm_count() * 8;
    // the queue kernel is instantiated per kind of id list: a bucket takes records only or none
    const bool queue_ok = queue && (qp[bucket].n_groups == 0 ||
                                    (qp[bucket].g[0].id_dtype == XB_REC64) == (h.id_dtype == XB_REC64));
    // likewise one instantiation per kind of id list for the short-segment kernel
    const bool short_ok = all_short && fast && d.tl == d.lpr &&
                          (hp[bucket].n_groups == 0 || (hp[bucket].g[0].id_dtype == XB_REC64) == (h.id_dtype == XB_REC64));
    PoolParams& dst = short_ok ? hp[bucket] : queue_ok ? qp[bucket] : fast ? fp[bucket] : p;
    d.warp_begin = dst.total_warps;
    const int spw = 32 / d.tl;
    const int64_t rounds = (h.batch + spw - 1) / spw;
    // the specialised kernel gives a warp several rounds, as long as every SM still gets dozens of warps
    d.segs = 1;
    if (fast) d.segs = (int)std::max<int64_t>(1, std::min<int64_t>(8, rounds / ((int64_t)sm_count() * 48)));
    // the short-segment kernel walks 8 rounds per warp (its prefetch needs a few), fewer only for small groups
    if (short_ok) d.segs = (int)std::max<int64_t>(1, std::min<int64_t>(8, rounds / ((int64_t)sm_count() * 16)));
    dst.total_warps += queue_ok && !short_ok ? (h.batch + 31) / 32 : (rounds + d.segs - 1) / d.segs;
    dst.g[dst.n_groups++] = d;
  }
  if (sp.n) {
    if (sp.chunk_begin[sp.n] > sp.n) {
      // some count array is longer than one chunk: all chunks in parallel, two launches
      scan_sums_kernel<<<sp.chunk_begin[sp.n], SCAN_THREADS, 0, stream>>>(sp);
      if (int rc = check_launch("scan_sums_kernel")) return rc;
      scan_apply_kernel<<<sp.chunk_begin[sp.n], SCAN_THREADS, 0, stream>>>(sp);
      if (int rc = check_launch("scan_apply_kernel")) return rc;
    } else {
      scan_counts_kernel<<<sp.n, SCAN_THREADS, 0, stream>>>(sp);
      if (int rc = check_launch("scan_counts_kernel")) return rc;
    }
  }
  for (int b = 0; b < kBuckets; ++b) {
    if (fp[b].n_groups == 0) continue;
    const int64_t blocks = (fp[b].total_warps + 7) / 8;
    XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_embedding_pool: too many segments");
    const int lpr = 2 << (b & 3);
    const int rc = b < 4 ? launch_pool_fast<XB_F32>(fp[b], lpr, (unsigned)blocks, stream)
                         : launch_pool_fast<XB_F16>(fp[b], lpr, (unsigned)blocks, stream);
    if (rc) return rc;
  }
  for (int b = 0; b < kBuckets; ++b) {
    if (hp[b].n_groups == 0) continue;
    const int64_t blocks = (hp[b].total_warps + 7) / 8;
    XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_embedding_pool: too many segments");
    const int lpr = 2 << (b & 3);
    const bool rec = hp[b].g[0].id_dtype == XB_REC64;
    const int rc = b < 4 ? (rec ? launch_pool_short<XB_F32, true>(hp[b], lpr, (unsigned)blocks, stream)
                                : launch_pool_short<XB_F32, false>(hp[b], lpr, (unsigned)blocks, stream))
                         : (rec ? launch_pool_short<XB_F16, true>(hp[b], lpr, (unsigned)blocks, stream)
                                : launch_pool_short<XB_F16, false>(hp[b], lpr, (unsigned)blocks, stream));
    if (rc) return rc;
  }
  for (int b = 0; b < kBuckets; ++b) {
    if (qp[b].n_groups == 0) continue;
    const int64_t blocks = (qp[b].total_warps + 7) / 8;
    XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_embedding_pool: too many segments");
    const int lpr = 2 << (b & 3);
    const bool rec = qp[b].g[0].id_dtype == XB_REC64;       // a queue bucket holds records only or none (see above)
    const int rc = b < 4 ? (rec ? launch_pool_queue<XB_F32, true>(qp[b], lpr, (unsigned)blocks, stream)
                                : launch_pool_queue<XB_F32, false>(qp[b], lpr, (unsigned)blocks, stream))
                         : (rec ? launch_pool_queue<XB_F16, true>(qp[b], lpr, (unsigned)blocks, stream)
                                : launch_pool_queue<XB_F16, false>(qp[b], lpr, (unsigned)blocks, stream));
    if (rc) return rc;
  }
  if (p.n_groups == 0) return 0;
  const int64_t blocks = (p.total_warps + 7) / 8;
  XB_REQUIRE(blocks < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_embedding_pool: too many segments");
  pool_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  return check_launch("pool_kernel");
}

// ---------------------------------------------------------------------------
// Measurement aid: the rate at which this GPU gathers rows at given (uniformly random) row numbers, with nothing
// else to do - four lanes per row, 16-byte loads, four rows in flight per lane. It is the ceiling a pooling kernel
// can reach on a table that does not fit L2, far below the streaming-copy bandwidth for 64-byte rows.
__global__ void __launch_bounds__(256) gather_probe_kernel(const uint4* __restrict__ table, int pitch16, int chunks,
                                                           const int32_t* __restrict__ rows, int64_t n, float* sink) {
  const int lane = threadIdx.x & 31, sub = lane >> 2, chunk = lane & 3;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t)gridDim.x * 8;
  float acc = 0.f;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    int r[4];
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) { const int64_t i = base + u * 8 + sub; r[u] = i < n ? __ldcs(rows + i) : -1; }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      v[u] = (r[u] >= 0 && chunk < chunks) ? __ldg(table + (int64_t)r[u] * pitch16 + chunk) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < 4; ++u) acc += __uint_as_float(v[u].x) + __uint_as_float(v[u].w);
  }
  if (acc == 12345.678f) sink[0] = acc;                // keeps the loads alive
}

extern "C" int xb_gather_probe(const xb_table_desc* table, const int32_t* row_ids, int64_t n, float* sink, xb_stream_t stream) {
  XB_REQUIRE(table && table->weights && row_ids && sink && n >= 0, XB_ERR_ARG, "xb_gather_probe: bad arguments");
  XB_REQUIRE(table->row_pitch_bytes % 16 == 0 && table->row_pitch_bytes <= 64, XB_ERR_LIMIT,
             "xb_gather_probe: rows of at most 64 bytes at a 16-byte pitch");
  const int esz = table->dtype == XB_F32 ? 4 : 2;
  const int chunks = (table->dim * esz + 15) / 16;
  gather_probe_kernel<<<sm_count() * 32, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint4*>(table->weights),
                                                                       (int)(table->row_pitch_bytes / 16), chunks, row_ids, n, sink);
  return check_launch("gather_probe_kernel");
}

// ---------------------------------------------------------------------------
// Allocation-free variant: the counts->offsets scratch lives in a file-scope
// device array instead of caller-provided memory.
#define XB_POOL_STATIC_SCRATCH_BYTES (1u << 20)
static __device__ __align__(256) unsigned char g_pool_static_scratch[XB_POOL_STATIC_SCRATCH_BYTES];

extern "C" size_t xb_embedding_pool_static_max_bytes(void) { return XB_POOL_STATIC_SCRATCH_BYTES; }

extern "C" int xb_embedding_pool_static(const xb_pool_group* groups, int32_t n_groups, xb_stream_t stream) {
  // In host code the array's name is only a handle; its device address has to be asked for,
  // once per device, while that device is current.
  // (threads that make the first call on a device at the same time all look up and store the same address)
  static std::atomic<void*> dev_ptr[64];
  int dev = -1;
  XB_CUDA(cudaGetDevice(&dev));
  XB_REQUIRE(dev >= 0 && dev < 64, XB_ERR_LIMIT, "xb_embedding_pool_static: device ordinal %d out of range", dev);
  if (dev_ptr[dev].load(std::memory_order_acquire) == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_pool_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(XB_ERR_CUDA, "xb_embedding_pool_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    dev_ptr[dev].store(p, std::memory_order_release);
  }
  XB_REQUIRE(groups && n_groups > 0, XB_ERR_ARG, "xb_embedding_pool_static: no groups");
  const size_t need = xb_embedding_pool_scratch_bytes(groups, n_groups);
  XB_REQUIRE(need <= XB_POOL_STATIC_SCRATCH_BYTES, XB_ERR_LIMIT,
             "xb_embedding_pool_static: these groups need %zu bytes of offset scratch, the built-in buffer holds %u "
             "(pass exclusive offsets instead of counts, split the call, or use xb_embedding_pool)",
             need, XB_POOL_STATIC_SCRATCH_BYTES);
  return xb_embedding_pool(groups, n_groups, dev_ptr[dev].load(std::memory_order_acquire), XB_POOL_STATIC_SCRATCH_BYTES,
                           stream);
}

// ---------------------------------------------------------------------------
// Row-sharded tables: routing of ids to their owner rank and the fixed-order
// combine of the partial pooled vectors that come back.
//
// Rule (the CPU restatement is orc_route): owner = (uint64)id % shards,
// local row = (uint64)id / shards. Ids are bucketed by owner with a STABLE
// counting sort (original order kept inside a bucket), so that the ids of one
// segment stay contiguous and ascending in segment number at the owner, and the
// whole exchange is reproducible bit for bit.
namespace xb {

constexpr int ROUTE_CHUNK = 4096;     // ids per CTA
constexpr int ROUTE_MAX_SHARDS = 16;

// owner = id % shards and local row = id / shards; a mask and a shift when shards is a power of two
__device__ __forceinline__ int route_owner(uint64_t id, int shards) {
  return (shards & (shards - 1)) == 0 ? (int)(id & (uint64_t)(shards - 1)) : (int)(id % (uint64_t)shards);
}
__device__ __forceinline__ uint64_t route_row(uint64_t id, int shards) {
  return (shards & (shards - 1)) == 0 ? id >> (31 - __clz(shards)) : id / (uint64_t)shards;
}
// last segment whose exclusive offset is <= idx, searched in [lo, hi)
__device__ __forceinline__ int64_t route_segment(const int32_t* __restrict__ seg_offsets, int64_t lo, int64_t hi, int64_t idx) {
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if ((int64_t)__ldg(seg_offsets + mid) <= idx) lo = mid; else hi = mid;
  }
  return lo;
}

// pass 1: per-CTA histogram of owners
// the segment of the first id of every scatter CTA (one search per thread); the entry after the last CTA closes the
// last window
__global__ void route_windows_kernel(const int32_t* __restrict__ seg_offsets, int64_t segments, int64_t n, int64_t blocks,
                                     int32_t* __restrict__ block_first_seg) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b > blocks) return;
  const int64_t first = b * ROUTE_CHUNK;
  const int32_t last_seg = (int32_t)(segments > 0 ? segments - 1 : 0);
  block_first_seg[b] = (b < blocks && first < n && segments > 0) ? (int32_t)route_segment(seg_offsets, 0, segments, first) : last_seg;
}

__global__ void __launch_bounds__(256) route_count_kernel(const int64_t* __restrict__ ids, int64_t n, int shards,
                                                          int32_t* __restrict__ block_hist) {
  __shared__ int32_t hist[ROUTE_MAX_SHARDS];
  if (threadIdx.x < ROUTE_MAX_SHARDS) hist[threadIdx.x] = 0;

  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * ROUTE_CHUNK;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < ROUTE_CHUNK; i += 256) {
    const int64_t idx = base + i;
    const int owner = idx < n ? route_owner((uint64_t)__ldcs(ids + idx), shards) : -1;
    // one shared-memory atomic per warp and owner instead of one per id (with two owners every id of a CTA would
    // queue on the same two words)
    for (int w = 0; w < shards; ++w) {
      const unsigned m = __ballot_sync(0xffffffffu, owner == w);
      if (lane == 0 && m) atomicAdd(&hist[w], __popc(m));                                // integer: order-free
    }
  }
  __syncthreads();
  if (threadIdx.x < shards) block_hist[(int64_t)blockIdx.x * shards + threadIdx.x] = hist[threadIdx.x];
}

// pass 2 (one CTA): exclusive scan in (owner, CTA) order -> first output slot of every (CTA, owner);
// owner_counts[w] = ids routed to w, owner_offsets[w] = start of bucket w
// With bucket_cap > 0 the buckets have a fixed capacity: bucket w starts at w * bucket_cap, its first slot holds
// the number of records that follow (the receiver reads it from there), and a bucket that would not fit sets
// *overflow and is cut at the capacity.
__global__ void __launch_bounds__(256) route_scan_kernel(int32_t* __restrict__ block_hist, int64_t blocks, int shards,
                                                         int64_t* __restrict__ owner_counts, int64_t bucket_cap,
                                                         int64_t* __restrict__ headers, int32_t* __restrict__ overflow) {
  __shared__ int64_t total_s;
  __shared__ int32_t part[256];
  if (threadIdx.x == 0) total_s = 0;
  __syncthreads();
  for (int w = 0; w < shards; ++w) {
    const int64_t start = total_s;
    for (int64_t b0 = 0; b0 < blocks; b0 += 256) {
      const int64_t b = b0 + threadIdx.x;
      const int32_t v = b < blocks ? block_hist[b * shards + w] : 0;
      part[threadIdx.x] = v;
      __syncthreads();
      // Hillis-Steele inclusive scan of the 256 partials
      for (int off = 1; off < 256; off <<= 1) {
        int32_t add = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
        __syncthreads();
        part[threadIdx.x] += add;
        __syncthreads();
      }
      if (b < blocks)
        block_hist[b * shards + w] = bucket_cap > 0 ? (int32_t)(w * bucket_cap + 1 + (total_s - start) + part[threadIdx.x] - v)
                                                    : (int32_t)(total_s + part[threadIdx.x] - v);
      __syncthreads();
      if (threadIdx.x == 255) total_s += part[255];
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      const int64_t cnt = total_s - start;
      if (owner_counts) owner_counts[w] = cnt;
      if (bucket_cap > 0) {
        headers[w * bucket_cap] = cnt < bucket_cap ? cnt : bucket_cap - 1;
        if (cnt >= bucket_cap) atomicExch(overflow, 1);
      }
    }
    __syncthreads();
  }
}

// pass 3: stable scatter. tags[i] is the segment number of id i (expanded from the counts by the caller's
// offsets: found here by binary search over the exclusive offsets).
__global__ void __launch_bounds__(256) route_scatter_kernel(const int64_t* __restrict__ ids, const float* __restrict__ values,
                                                            const int32_t* __restrict__ seg_offsets, int64_t segments,
                                                            int64_t n, int shards, const int32_t* __restrict__ block_base,
                                                            int64_t* __restrict__ out_rows, float* __restrict__ out_values,
                                                            int32_t* __restrict__ out_tags, int64_t bucket_cap,
                                                            const int32_t* __restrict__ block_first_seg) {
  // The kernel is bound by instructions per id, not by memory, so the per-id work is kept to a handful: the segment
  // of every id of the CTA is tabulated once in shared memory (each segment of the CTA's window writes its number
  // over its own positions), and the ranks come from prefix sums that `shards` threads make once per round.
  constexpr int RK = 4;                                       // sub-rounds of 256 ids per round
  constexpr int WIN = 65536;                                  // the table holds 16-bit segment numbers relative to the window
  __shared__ int32_t running[2][ROUTE_MAX_SHARDS];
  __shared__ int32_t warp_cnt[2][RK][8][ROUTE_MAX_SHARDS];     // counts, then exclusive prefixes in (sub-round, warp) order
  __shared__ __align__(16) uint16_t seg_rel[ROUTE_CHUNK];
  const int64_t base = (int64_t)blockIdx.x * ROUTE_CHUNK;
  if (threadIdx.x < shards) running[0][threadIdx.x] = block_base[(int64_t)blockIdx.x * shards + threadIdx.x];
  // the ids of this CTA are consecutive, so their segments lie between the segment of its first id and that of
  // the next CTA's first id (both found by route_windows_kernel)
  const int64_t win_lo = __ldg(block_first_seg + blockIdx.x), win_hi = (int64_t)__ldg(block_first_seg + blockIdx.x + 1) + 1;
  const bool tabulated = win_hi - win_lo <= WIN;              // otherwise (mostly empty segments) every id searches the offsets
  if (tabulated) {
    // positions no segment claims (ids past the last offset) get the window's last segment, as the search would give
    const uint32_t fill = (uint32_t)(win_hi - 1 - win_lo) * 0x00010001u;
    for (int i = threadIdx.x; i < ROUTE_CHUNK / 8; i += 256) reinterpret_cast<uint4*>(seg_rel)[i] = make_uint4(fill, fill, fill, fill);
    __syncthreads();
    const int64_t end = min(base + (int64_t)ROUTE_CHUNK, n);
    for (int64_t sgm = win_lo + threadIdx.x; sgm < win_hi; sgm += 256) {
      const int64_t p0 = max((int64_t)__ldg(seg_offsets + sgm), base), p1 = min((int64_t)__ldg(seg_offsets + sgm + 1), end);
      for (int64_t pp = p0; pp < p1; ++pp) seg_rel[pp - base] = (uint16_t)(sgm - win_lo);
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Rounds of RK x 256 consecutive ids: thread t takes the ids t, t + 256, ... of a round, so every load and (per
  // owner) every store is coalesced and all RK loads are in flight together. The ranking stays stable: an id is
  // preceded by the ids of earlier rounds, of earlier sub-rounds, of lower warps in its sub-round and of lower lanes
  // in its warp.
  for (int i0 = 0, rnd = 0; i0 < ROUTE_CHUNK; i0 += RK * 256, rnd ^= 1) {
    uint64_t id[RK];
    int owner[RK], rank_in_warp[RK];
#pragma unroll
    for (int k = 0; k < RK; ++k) {
      const int64_t idx = base + i0 + k * 256 + threadIdx.x;
      id[k] = idx < n ? (uint64_t)__ldcs(ids + idx) : 0;
    }
#pragma unroll
    for (int k = 0; k < RK; ++k) {
      const int64_t idx = base + i0 + k * 256 + threadIdx.x;
      owner[k] = idx < n ? route_owner(id[k], shards) : -1;
      rank_in_warp[k] = 0;
      for (int w = 0; w < shards; ++w) {
        const unsigned m = __ballot_sync(0xffffffffu, owner[k] == w);
        if (owner[k] == w) rank_in_warp[k] = __popc(m & ((1u << lane) - 1));
        if (lane == 0) warp_cnt[rnd][k][warp][w] = __popc(m);
      }
    }
    __syncthreads();                                          // the counts of this round are written
    if (threadIdx.x < shards) {
      // counts -> exclusive prefixes in (sub-round, warp) order, starting from the ids of the rounds before
      int acc = running[rnd][threadIdx.x];
      for (int k = 0; k < RK; ++k)
        for (int ww = 0; ww < 8; ++ww) {
          const int c = warp_cnt[rnd][k][ww][threadIdx.x];
          warp_cnt[rnd][k][ww][threadIdx.x] = acc;
          acc += c;
        }
      running[rnd ^ 1][threadIdx.x] = acc;
    }
    __syncthreads();                                          // the prefixes are written
#pragma unroll
    for (int k = 0; k < RK; ++k) {
      const int64_t idx = base + i0 + k * 256 + threadIdx.x;
      if (idx < n) {
        const int ow = owner[k];
        const int64_t pos = (int64_t)warp_cnt[rnd][k][warp][ow] + rank_in_warp[k];
        // segment of this id: last offset <= idx
        const int64_t lo = tabulated ? win_lo + seg_rel[i0 + k * 256 + threadIdx.x] : route_segment(seg_offsets, win_lo, win_hi, idx);
        const uint64_t row = route_row(id[k], shards);
        if (bucket_cap > 0 && pos >= (int64_t)(ow + 1) * bucket_cap) {
          // beyond the bucket's capacity: dropped (route_scan_kernel has raised the overflow flag)
        } else if (out_tags) {
          out_rows[pos] = (int64_t)row;
          out_tags[pos] = (int32_t)lo;
        } else {
          // packed record: segment number in the high half, local row in the low half; a row that does not
          // fit 31 bits cannot exist in a shard and is sent as 0x7fffffff, which no shard holds either
          out_rows[pos] = (int64_t)(((uint64_t)lo << 32) | (row < 0x7fffffffull ? row : 0x7fffffffull));
        }
        if (out_values && bucket_cap == 0) out_values[pos] = values ? values[idx] : 1.f;
      }
    }
    // the next round counts into the other buffer and reads the other `running`; two rounds on, every thread has
    // passed two more barriers, so nothing of this round is still being read when its buffer is written again
  }
}

// packed records (see route_scatter_kernel) -> int32 local rows and int32 segment numbers
__global__ void unpack_routed_kernel(const int64_t* __restrict__ packed, int64_t n, int32_t* __restrict__ rows,
                                     int32_t* __restrict__ tags) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t v = (uint64_t)__ldcs(packed + i);
    rows[i] = (int32_t)(v & 0xffffffffull);
    tags[i] = (int32_t)(v >> 32);
  }
}

// segment lengths of everything an owner received, all source ranks in one launch: slice s of the tags
// (bounds[s] .. bounds[s+1]) counts into counts[s * segments + tag]
struct TagBounds { int64_t b[ROUTE_MAX_SHARDS + 1]; };
__global__ void tag_count_sources_kernel(const int32_t* __restrict__ tags, const TagBounds bounds, int sources,
                                         int64_t segments, int32_t* __restrict__ counts) {
  const int64_t n = bounds.b[sources];
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int src = 0;
    while (src + 1 < sources && i >= bounds.b[src + 1]) ++src;
    // a tag comes from a peer: one outside [0, segments) is dropped, never used as an index
    const uint32_t tag = (uint32_t)tags[i];
    if (tag < (uint64_t)segments) atomicAdd(&counts[(int64_t)src * segments + tag], 1);
  }
}

// segment lengths at the owner: tags arrive sorted per source rank; counts are integer atomics (exact)
__global__ void tag_count_kernel(const int32_t* __restrict__ tags, int64_t n, int32_t* __restrict__ counts,
                                 int64_t n_counts) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t tag = (uint32_t)tags[i];
    if (tag < (uint64_t)n_counts) atomicAdd(&counts[tag], 1);
  }
}

// out[s, col0 + e] = scale(s) * sum_{w=0..shards-1} partial[w][s][e], w ascending (fixed order)
__global__ void shard_combine_kernel(const float* __restrict__ partial, int shards, int64_t segments, int dim,
                                     const int32_t* __restrict__ seg_len, int avg, void* out, int64_t out_stride,
                                     int64_t seg_per_row, int out_dtype) {
  const int64_t total = segments * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / dim;
    const int e = (int)(i - s * dim);
    float acc = 0.f;
    for (int w = 0; w < shards; ++w) acc += partial[((int64_t)w * segments + s) * dim + e];
    if (avg && seg_len && seg_len[s] != 0) acc = acc * (float)(1.0 / (double)seg_len[s]);
    // segment s = group * rows + sample  ->  out[sample, group*dim + e]
    const int64_t rows = segments / seg_per_row;
    const int64_t grp = s / rows, sample = s - grp * rows;
    store_out(out, sample * out_stride + grp * dim + e, out_dtype, acc);
  }
}

// The same sum, four adjacent elements per thread (dim and the output row stride multiples of 4, aligned
// bases): 16-byte loads of all owners' partials are issued before the first add, the adds keep the owner order.
template <int SHARDS>
__global__ void __launch_bounds__(256) shard_combine4_kernel(const float4* __restrict__ partial, int shards, int64_t segments,
                                                             int dim4, const int32_t* __restrict__ seg_len, int avg,
                                                             void* out, int64_t out_stride, int64_t rows, int out_dtype) {
  const int64_t total = segments * dim4;
  const int n_sh = SHARDS ? SHARDS : shards;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / dim4;
    const int e4 = (int)(i - s * dim4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (SHARDS) {
      float4 v[SHARDS ? SHARDS : 1];
#pragma unroll
      for (int w = 0; w < SHARDS; ++w) v[w] = __ldcs(partial + ((int64_t)w * segments + s) * dim4 + e4);
#pragma unroll
      for (int w = 0; w < SHARDS; ++w) { acc.x += v[w].x; acc.y += v[w].y; acc.z += v[w].z; acc.w += v[w].w; }
    } else {
      for (int w = 0; w < n_sh; ++w) {
        const float4 v = __ldcs(partial + ((int64_t)w * segments + s) * dim4 + e4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    if (avg && seg_len) {
      const int32_t len = seg_len[s];
      if (len != 0) {
        const float sc = (float)(1.0 / (double)len);
        acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
      }
    }
    // segment s = group * rows + sample  ->  out[sample, group*dim + e]
    const int64_t grp = s / rows, sample = s - grp * rows;
    const int64_t o = sample * out_stride + (grp * dim4 + e4) * 4;
    if (out_dtype == XB_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = acc;
    } else {
      const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + o) =
          make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
  }
}

// Partial sums that crossed the wire as fp16 (a model whose tables and activations are fp16): eight adjacent
// elements per thread, one 16-byte load per owner, fp32 accumulation in owner order.
template <int SHARDS>
__global__ void __launch_bounds__(256) shard_combine_h8_kernel(const uint4* __restrict__ partial, int shards, int64_t segments,
                                                               int dim8, const int32_t* __restrict__ seg_len, int avg,
                                                               void* out, int64_t out_stride, int64_t rows, int out_dtype) {
  const int64_t total = segments * dim8;
  const int n_sh = SHARDS ? SHARDS : shards;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / dim8;
    const int e8 = (int)(i - s * dim8);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    auto add = [&](const uint4& v) {
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        acc[2 * e] += f.x; acc[2 * e + 1] += f.y;
      }
    };
    if (SHARDS) {
      uint4 v[SHARDS ? SHARDS : 1];
#pragma unroll
      for (int w = 0; w < SHARDS; ++w) v[w] = __ldcs(partial + ((int64_t)w * segments + s) * dim8 + e8);
#pragma unroll
      for (int w = 0; w < SHARDS; ++w) add(v[w]);
    } else {
      for (int w = 0; w < n_sh; ++w) add(__ldcs(partial + ((int64_t)w * segments + s) * dim8 + e8));
    }
    if (avg && seg_len) {
      const int32_t len = seg_len[s];
      if (len != 0) {
        const float sc = (float)(1.0 / (double)len);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] *= sc;
      }
    }
    const int64_t grp = s / rows, sample = s - grp * rows;
    const int64_t o = sample * out_stride + (grp * dim8 + e8) * 8;
    if (out_dtype == XB_F32) {
      float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o);
      d[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      d[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint4 r;
      __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
      *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out) + o) = r;
    }
  }
}

// fp16 partials of any shape, one element per thread
__global__ void shard_combine_h_kernel(const __half* __restrict__ partial, int shards, int64_t segments, int dim,
                                       const int32_t* __restrict__ seg_len, int avg, void* out, int64_t out_stride,
                                       int64_t seg_per_row, int out_dtype) {
  const int64_t total = segments * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / dim;
    const int e = (int)(i - s * dim);
    float acc = 0.f;
    for (int w = 0; w < shards; ++w) acc += __half2float(partial[((int64_t)w * segments + s) * dim + e]);
    if (avg && seg_len && seg_len[s] != 0) acc = acc * (float)(1.0 / (double)seg_len[s]);
    const int64_t rows = segments / seg_per_row;
    const int64_t grp = s / rows, sample = s - grp * rows;
    store_out(out, sample * out_stride + grp * dim + e, out_dtype, acc);
  }
}

}  // namespace xb

extern "C" size_t xb_route_scratch_bytes(int64_t n_ids, int32_t shards) {
  const int64_t blocks = std::max<int64_t>((n_ids + ROUTE_CHUNK - 1) / ROUTE_CHUNK, 1);
  // per-CTA owner histogram, then the first segment of every CTA's ids (one more entry closes the last window)
  return (size_t)blocks * shards * sizeof(int32_t) + (size_t)(blocks + 1) * sizeof(int32_t);
}

extern "C" int xb_route_ids(const int64_t* ids, const float* values, const int32_t* seg_offsets, int64_t segments,
                            int64_t n_ids, int32_t shards, int64_t* out_rows, float* out_values, int32_t* out_tags,
                            int64_t* owner_counts, void* scratch, size_t scratch_bytes, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(shards >= 1 && shards <= ROUTE_MAX_SHARDS, XB_ERR_LIMIT, "xb_route_ids: %d shards (1..%d)", shards, ROUTE_MAX_SHARDS);
  XB_REQUIRE(n_ids >= 0 && segments >= 0 && owner_counts && out_rows && seg_offsets, XB_ERR_ARG, "xb_route_ids: bad arguments");
  XB_REQUIRE(out_tags || segments < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_route_ids: packed records hold 31-bit segment numbers");
  XB_REQUIRE(n_ids == 0 || ids, XB_ERR_ARG, "xb_route_ids: ids missing");
  XB_REQUIRE(n_ids < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_route_ids: more than 2^31 ids per call");
  XB_REQUIRE(scratch_bytes >= xb_route_scratch_bytes(n_ids, shards) && scratch, XB_ERR_SCRATCH, "xb_route_ids: scratch too small");
  const int64_t blocks = std::max<int64_t>((n_ids + ROUTE_CHUNK - 1) / ROUTE_CHUNK, 1);
  int32_t* hist = reinterpret_cast<int32_t*>(scratch);
  int32_t* first_seg = hist + blocks * shards;
  route_count_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ids, n_ids, shards, hist);
  route_windows_kernel<<<(unsigned)((blocks + 256) / 256), 256, 0, stream>>>(seg_offsets, segments, n_ids, blocks, first_seg);
  route_scan_kernel<<<1, 256, 0, stream>>>(hist, blocks, shards, owner_counts, 0, nullptr, nullptr);
  route_scatter_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ids, values, seg_offsets, segments, n_ids, shards, hist, out_rows,
                                                             out_values, out_tags, 0, first_seg);
  return check_launch("route kernels");
}

extern "C" int xb_route_ids_padded(const int64_t* ids, const int32_t* seg_offsets, int64_t segments, int64_t n_ids,
                                   int32_t shards, int64_t bucket_cap, int64_t* out_records, int32_t* overflow,
                                   void* scratch, size_t scratch_bytes, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(shards >= 1 && shards <= ROUTE_MAX_SHARDS, XB_ERR_LIMIT, "xb_route_ids_padded: %d shards (1..%d)", shards, ROUTE_MAX_SHARDS);
  XB_REQUIRE(n_ids >= 0 && segments >= 0 && out_records && seg_offsets && overflow, XB_ERR_ARG, "xb_route_ids_padded: bad arguments");
  XB_REQUIRE(segments < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_route_ids_padded: packed records hold 31-bit segment numbers");
  XB_REQUIRE(n_ids == 0 || ids, XB_ERR_ARG, "xb_route_ids_padded: ids missing");
  XB_REQUIRE(bucket_cap >= 2 && bucket_cap * shards < ((int64_t)1 << 31), XB_ERR_LIMIT,
             "xb_route_ids_padded: bucket capacity %lld (2 .. 2^31 / shards)", (long long)bucket_cap);
  XB_REQUIRE(n_ids < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_route_ids_padded: more than 2^31 ids per call");
  XB_REQUIRE(scratch_bytes >= xb_route_scratch_bytes(n_ids, shards) && scratch, XB_ERR_SCRATCH, "xb_route_ids_padded: scratch too small");
  const int64_t blocks = std::max<int64_t>((n_ids + ROUTE_CHUNK - 1) / ROUTE_CHUNK, 1);
  int32_t* hist = reinterpret_cast<int32_t*>(scratch);
  int32_t* first_seg = hist + blocks * shards;
  route_count_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ids, n_ids, shards, hist);
  route_windows_kernel<<<(unsigned)((blocks + 256) / 256), 256, 0, stream>>>(seg_offsets, segments, n_ids, blocks, first_seg);
  route_scan_kernel<<<1, 256, 0, stream>>>(hist, blocks, shards, nullptr, bucket_cap, out_records, overflow);
  route_scatter_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ids, nullptr, seg_offsets, segments, n_ids, shards, hist, out_records,
                                                             nullptr, nullptr, bucket_cap, first_seg);
  return check_launch("route kernels (fixed-capacity buckets)");
}

// fixed-capacity buckets as received: slot 0 of every bucket is its record count; slots past the count get tag -1
__global__ void unpack_padded_kernel(const int64_t* __restrict__ packed, int sources, int64_t cap, int32_t* __restrict__ rows,
                                     int32_t* __restrict__ tags) {
  const int64_t n = (int64_t)sources * cap;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = i / cap, j = i - s * cap;
    int64_t cnt = __ldg(packed + s * cap);
    cnt = cnt < 0 ? 0 : (cnt > cap - 1 ? cap - 1 : cnt);          // the header comes from a peer: bounded here
    const bool live = j >= 1 && j <= cnt;
    const uint64_t v = live ? (uint64_t)__ldcs(packed + i) : 0ull;
    rows[i] = (int32_t)(v & 0xffffffffull);
    tags[i] = live ? (int32_t)(v >> 32) : -1;
  }
}

extern "C" int xb_unpack_routed_padded(const int64_t* packed, int32_t sources, int64_t bucket_cap, int32_t* rows, int32_t* tags,
                                       xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(packed && rows && tags && sources >= 1 && bucket_cap >= 2, XB_ERR_ARG, "xb_unpack_routed_padded: bad arguments");
  const int64_t n = (int64_t)sources * bucket_cap;
  const int64_t blocks = std::min<int64_t>((n + 255) / 256, (int64_t)sm_count() * 16);
  unpack_padded_kernel<<<(unsigned)blocks, 256, 0, stream>>>(packed, sources, bucket_cap, rows, tags);
  return check_launch("unpack_padded_kernel");
}

extern "C" size_t xb_scan_counts_scratch_bytes(int32_t n_arrays, int64_t batch) {
  return (size_t)n_arrays * align256(scan_chunks(batch) * 4);
}

extern "C" int xb_scan_counts(const int32_t* counts, int64_t counts_stride, int32_t* offsets, int64_t offsets_stride,
                              int32_t n_arrays, int64_t batch, void* scratch, size_t scratch_bytes, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(counts && offsets && n_arrays >= 1 && n_arrays <= XB_MAX_POOL_GROUPS && batch >= 0, XB_ERR_ARG,
             "xb_scan_counts: bad arguments (1..%d arrays)", XB_MAX_POOL_GROUPS);
  XB_REQUIRE(scratch && scratch_bytes >= xb_scan_counts_scratch_bytes(n_arrays, batch), XB_ERR_SCRATCH, "xb_scan_counts: scratch too small");
  static thread_local ScanParams sp;
  sp.n = n_arrays;
  sp.chunk_begin[0] = 0;
  const size_t per = align256(scan_chunks(batch) * 4);
  for (int i = 0; i < n_arrays; ++i) {
    sp.counts[i] = counts + (int64_t)i * counts_stride;
    sp.offsets[i] = offsets + (int64_t)i * offsets_stride;
    sp.batch[i] = batch;
    sp.chunk_sums[i] = reinterpret_cast<int32_t*>((char*)scratch + i * per);
    sp.chunk_begin[i + 1] = sp.chunk_begin[i] + (int32_t)scan_chunks(batch);
  }
  if (batch == 0) return 0;
  if (sp.chunk_begin[sp.n] > sp.n) {
    scan_sums_kernel<<<sp.chunk_begin[sp.n], SCAN_THREADS, 0, stream>>>(sp);
    if (int rc = check_launch("scan_sums_kernel")) return rc;
    scan_apply_kernel<<<sp.chunk_begin[sp.n], SCAN_THREADS, 0, stream>>>(sp);
    return check_launch("scan_apply_kernel");
  }
  scan_counts_kernel<<<sp.n, SCAN_THREADS, 0, stream>>>(sp);
  return check_launch("scan_counts_kernel");
}

extern "C" int xb_unpack_routed(const int64_t* packed, int64_t n, int32_t* rows, int32_t* tags, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(n >= 0 && (n == 0 || (packed && rows && tags)), XB_ERR_ARG, "xb_unpack_routed: bad arguments");
  if (n == 0) return 0;
  const int64_t blocks = std::min<int64_t>((n + 255) / 256, (int64_t)sm_count() * 16);
  unpack_routed_kernel<<<(unsigned)blocks, 256, 0, stream>>>(packed, n, rows, tags);
  return check_launch("unpack_routed_kernel");
}

extern "C" int xb_tag_counts(const int32_t* tags, int64_t n, int32_t* counts, int64_t n_counts, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(counts && n >= 0 && n_counts >= 0 && (n == 0 || tags), XB_ERR_ARG, "xb_tag_counts: bad arguments");
  XB_CUDA(cudaMemsetAsync(counts, 0, (size_t)n_counts * sizeof(int32_t), stream));
  if (n == 0) return 0;
  const int64_t blocks = std::min<int64_t>((n + 255) / 256, (int64_t)sm_count() * 8);
  tag_count_kernel<<<(unsigned)blocks, 256, 0, stream>>>(tags, n, counts, n_counts);
  return check_launch("tag_count_kernel");
}

extern "C" int xb_tag_counts_sources(const int32_t* tags, const int64_t* source_counts, int32_t sources, int32_t* counts,
                                     int64_t segments, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(source_counts && counts && segments >= 0, XB_ERR_ARG, "xb_tag_counts_sources: bad arguments");
  XB_REQUIRE(sources >= 1 && sources <= ROUTE_MAX_SHARDS, XB_ERR_LIMIT, "xb_tag_counts_sources: %d sources (1..%d)", sources, ROUTE_MAX_SHARDS);
  TagBounds bounds;
  bounds.b[0] = 0;
  for (int s = 0; s < sources; ++s) {
    XB_REQUIRE(source_counts[s] >= 0, XB_ERR_ARG, "xb_tag_counts_sources: negative count");
    bounds.b[s + 1] = bounds.b[s] + source_counts[s];
  }
  const int64_t n = bounds.b[sources];
  XB_REQUIRE(n == 0 || tags, XB_ERR_ARG, "xb_tag_counts_sources: tags missing");
  XB_CUDA(cudaMemsetAsync(counts, 0, (size_t)sources * (size_t)segments * sizeof(int32_t), stream));
  if (n == 0) return 0;
  const int64_t blocks = std::min<int64_t>((n + 255) / 256, (int64_t)sm_count() * 8);
  tag_count_sources_kernel<<<(unsigned)blocks, 256, 0, stream>>>(tags, bounds, sources, segments, counts);
  return check_launch("tag_count_sources_kernel");
}

extern "C" int xb_shard_pool(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                             const void* rows, int32_t row_dtype, int64_t n_rows, const float* values,
                             const int32_t* offsets, int32_t sources, int32_t dim, void* out, int32_t out_dtype,
                             xb_stream_t stream) {
  XB_REQUIRE(tables && table_segments && n_tables >= 1 && sources >= 1 && offsets && out && dim >= 1, XB_ERR_ARG,
             "xb_shard_pool: bad arguments");
  XB_REQUIRE(out_dtype == XB_F32 || out_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_pool: partial dtype %d", out_dtype);
  const size_t out_esz = out_dtype == XB_F32 ? 4 : 2;
  int64_t S = 0;
  for (int t = 0; t < n_tables; ++t) {
    XB_REQUIRE(table_segments[t] >= 0, XB_ERR_ARG, "xb_shard_pool: negative segment count");
    S += table_segments[t];
  }
  xb_pool_group groups[XB_MAX_POOL_GROUPS];
  int n = 0;
  for (int s = 0; s < sources; ++s) {
    int64_t lo = (int64_t)s * S;
    for (int t = 0; t < n_tables; ++t) {
      xb_pool_group& g = groups[n];
      memset(&g, 0, sizeof(g));
      g.table = tables[t];
      g.ids = rows;
      g.values = values;
      g.segments = offsets + lo;
      g.segments_are_offsets = 1;
      g.batch = table_segments[t];
      // the exact share of this (source, table) is only known on the device; it sizes the work split only
      g.n_ids = sources * S ? n_rows * table_segments[t] / ((int64_t)sources * S) : 0;
      g.dim = dim;
      g.id_dtype = row_dtype;
      g.out_dtype = out_dtype;
      g.n_items = 1;
      g.items[0].udf = XB_UDF_SUM;
      g.items[0].out = reinterpret_cast<char*>(out) + (size_t)lo * dim * out_esz;
      g.items[0].stride = dim;
      lo += table_segments[t];
      if (++n == XB_MAX_POOL_GROUPS) {
        if (int rc = xb_embedding_pool(groups, n, nullptr, 0, stream)) return rc;
        n = 0;
      }
    }
  }
  return n ? xb_embedding_pool(groups, n, nullptr, 0, stream) : 0;
}

extern "C" int xb_shard_pool_padded(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                                    const int32_t* rows, int64_t bucket_cap, const int32_t* offsets, int32_t sources,
                                    int64_t n_rows_estimate, int32_t dim, void* out, int32_t out_dtype, xb_stream_t stream) {
  XB_REQUIRE(tables && table_segments && n_tables >= 1 && sources >= 1 && offsets && rows && out && dim >= 1 && bucket_cap >= 2,
             XB_ERR_ARG, "xb_shard_pool_padded: bad arguments");
  XB_REQUIRE(out_dtype == XB_F32 || out_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_pool_padded: partial dtype %d", out_dtype);
  const size_t out_esz = out_dtype == XB_F32 ? 4 : 2;
  int64_t S = 0;
  for (int t = 0; t < n_tables; ++t) {
    XB_REQUIRE(table_segments[t] >= 0, XB_ERR_ARG, "xb_shard_pool_padded: negative segment count");
    S += table_segments[t];
  }
  xb_pool_group groups[XB_MAX_POOL_GROUPS];
  int n = 0;
  for (int s = 0; s < sources; ++s) {
    int64_t lo = 0;
    for (int t = 0; t < n_tables; ++t) {
      xb_pool_group& g = groups[n];
      memset(&g, 0, sizeof(g));
      g.table = tables[t];
      g.ids = rows + (int64_t)s * bucket_cap + 1;            // the records of source s follow its header slot
      g.segments = offsets + (int64_t)s * (S + 1) + lo;      // offsets of source s count from its first record
      g.segments_are_offsets = 1;
      g.batch = table_segments[t];
      g.n_ids = sources * S ? n_rows_estimate * table_segments[t] / ((int64_t)sources * S) : 0;   // sizes the work split only
      g.dim = dim;
      g.id_dtype = XB_I32;
      g.out_dtype = out_dtype;
      g.n_items = 1;
      g.items[0].udf = XB_UDF_SUM;
      g.items[0].out = reinterpret_cast<char*>(out) + ((size_t)s * S + lo) * dim * out_esz;
      g.items[0].stride = dim;
      lo += table_segments[t];
      if (++n == XB_MAX_POOL_GROUPS) {
        if (int rc = xb_embedding_pool(groups, n, nullptr, 0, stream)) return rc;
        n = 0;
      }
    }
  }
  return n ? xb_embedding_pool(groups, n, nullptr, 0, stream) : 0;
}

// Segment lengths at the owner straight from the received fixed-capacity buckets (no unpacked copy): slot 0 of a
// bucket is its record count, records arrive sorted by segment within a source, so the lanes of a warp that hold the
// same segment number add once. counts[src * segments + tag]; a tag outside [0, segments) is dropped.
__global__ void record_count_kernel(const int64_t* __restrict__ packed, int sources, int64_t cap, int64_t segments,
                                    int32_t* __restrict__ counts) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  for (int src = 0; src < sources; ++src) {
    int64_t cnt = __ldg(packed + (int64_t)src * cap);
    cnt = cnt < 0 ? 0 : (cnt > cap - 1 ? cap - 1 : cnt);            // the header comes from a peer: bounded here
    const int64_t rounds = (cnt + nthreads - 1) / nthreads;         // the same for every thread: whole warps stay together
    for (int64_t r = 0; r < rounds; ++r) {
      const int64_t j = r * nthreads + tid;
      uint32_t tag = 0xffffffffu;
      if (j < cnt) tag = (uint32_t)((uint64_t)__ldcs(packed + (int64_t)src * cap + 1 + j) >> 32);
      const unsigned same = __match_any_sync(0xffffffffu, tag);
      if (tag < (uint64_t)segments && (same & ((1u << lane) - 1)) == 0)
        atomicAdd(&counts[(int64_t)src * segments + tag], __popc(same));
    }
  }
}

extern "C" int xb_record_counts_padded(const int64_t* packed, int32_t sources, int64_t bucket_cap, int32_t* counts,
                                       int64_t segments, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(packed && counts && sources >= 1 && sources <= ROUTE_MAX_SHARDS && bucket_cap >= 2 && segments >= 0, XB_ERR_ARG,
             "xb_record_counts_padded: bad arguments");
  XB_CUDA(cudaMemsetAsync(counts, 0, (size_t)sources * (size_t)segments * sizeof(int32_t), stream));
  record_count_kernel<<<sm_count() * 8, 256, 0, stream>>>(packed, sources, bucket_cap, segments, counts);
  return check_launch("record_count_kernel");
}

// xb_shard_pool_padded reading the received records themselves (id dtype XB_REC64: the row is the low 32 bits).
extern "C" int xb_shard_pool_records(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                                     const int64_t* records, int64_t bucket_cap, const int32_t* offsets, int32_t sources,
                                     int64_t n_rows_estimate, int32_t dim, void* out, int32_t out_dtype, xb_stream_t stream) {
  XB_REQUIRE(tables && table_segments && n_tables >= 1 && sources >= 1 && offsets && records && out && dim >= 1 && bucket_cap >= 2,
             XB_ERR_ARG, "xb_shard_pool_records: bad arguments");
  XB_REQUIRE(out_dtype == XB_F32 || out_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_pool_records: partial dtype %d", out_dtype);
  const size_t out_esz = out_dtype == XB_F32 ? 4 : 2;
  int64_t S = 0;
  for (int t = 0; t < n_tables; ++t) {
    XB_REQUIRE(table_segments[t] >= 0, XB_ERR_ARG, "xb_shard_pool_records: negative segment count");
    S += table_segments[t];
  }
  xb_pool_group groups[XB_MAX_POOL_GROUPS];
  int n = 0;
  for (int s = 0; s < sources; ++s) {
    int64_t lo = 0;
    for (int t = 0; t < n_tables; ++t) {
      xb_pool_group& g = groups[n];
      memset(&g, 0, sizeof(g));
      g.table = tables[t];
      g.ids = records + (int64_t)s * bucket_cap + 1;         // the records of source s follow its header slot
      g.segments = offsets + (int64_t)s * (S + 1) + lo;      // offsets of source s count from its first record
      g.segments_are_offsets = 1;
      g.batch = table_segments[t];
      g.n_ids = sources * S ? n_rows_estimate * table_segments[t] / ((int64_t)sources * S) : 0;   // sizes the work split only
      g.dim = dim;
      g.id_dtype = XB_REC64;
      g.out_dtype = out_dtype;
      g.n_items = 1;
      g.items[0].udf = XB_UDF_SUM;
      g.items[0].out = reinterpret_cast<char*>(out) + ((size_t)s * S + lo) * dim * out_esz;
      g.items[0].stride = dim;
      lo += table_segments[t];
      if (++n == XB_MAX_POOL_GROUPS) {
        if (int rc = xb_embedding_pool(groups, n, nullptr, 0, stream)) return rc;
        n = 0;
      }
    }
  }
  return n ? xb_embedding_pool(groups, n, nullptr, 0, stream) : 0;
}

extern "C" int xb_shard_combine(const void* partial_, int32_t partial_dtype, int32_t shards, int64_t segments, int32_t dim,
                                const int32_t* seg_len, int32_t avg, void* out, int64_t out_stride, int64_t groups,
                                int32_t out_dtype, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(partial_dtype == XB_F32 || partial_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_combine: partial dtype %d",
             partial_dtype);
  if (partial_dtype == XB_F16) {
    XB_REQUIRE(partial_ && out && shards >= 1 && segments >= 0 && dim >= 1 && groups >= 1, XB_ERR_ARG, "xb_shard_combine: bad arguments");
    XB_REQUIRE(segments % groups == 0, XB_ERR_ARG, "xb_shard_combine: segments %lld not a multiple of groups %lld", (long long)segments, (long long)groups);
    XB_REQUIRE(out_dtype == XB_F32 || out_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_combine: output dtype %d", out_dtype);
    if (segments == 0) return 0;
    const size_t esz = out_dtype == XB_F32 ? 4 : 2;
    if (dim % 8 == 0 && out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(partial_) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & (8 * esz - 1) & 15) == 0) {
      const int dim8 = dim / 8;
      const int64_t rows = segments / groups;
      const int64_t blocks8 = std::min<int64_t>((segments * dim8 + 255) / 256, (int64_t)sm_count() * 16);
      const uint4* p8 = reinterpret_cast<const uint4*>(partial_);
      switch (shards) {
        case 2: shard_combine_h8_kernel<2><<<(unsigned)blocks8, 256, 0, stream>>>(p8, shards, segments, dim8, seg_len, avg, out, out_stride, rows, out_dtype); break;
        case 4: shard_combine_h8_kernel<4><<<(unsigned)blocks8, 256, 0, stream>>>(p8, shards, segments, dim8, seg_len, avg, out, out_stride, rows, out_dtype); break;
        case 8: shard_combine_h8_kernel<8><<<(unsigned)blocks8, 256, 0, stream>>>(p8, shards, segments, dim8, seg_len, avg, out, out_stride, rows, out_dtype); break;
        default: shard_combine_h8_kernel<0><<<(unsigned)blocks8, 256, 0, stream>>>(p8, shards, segments, dim8, seg_len, avg, out, out_stride, rows, out_dtype); break;
      }
      return check_launch("shard_combine_h8_kernel");
    }
    const int64_t blocks = std::min<int64_t>((segments * dim + 255) / 256, (int64_t)sm_count() * 8);
    shard_combine_h_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const __half*>(partial_), shards, segments, dim,
                                                                 seg_len, avg, out, out_stride, groups, out_dtype);
    return check_launch("shard_combine_h_kernel");
  }
  const float* partial = reinterpret_cast<const float*>(partial_);
  XB_REQUIRE(partial && out && shards >= 1 && segments >= 0 && dim >= 1 && groups >= 1, XB_ERR_ARG, "xb_shard_combine: bad arguments");
  XB_REQUIRE(segments % groups == 0, XB_ERR_ARG, "xb_shard_combine: segments %lld not a multiple of groups %lld", (long long)segments, (long long)groups);
  XB_REQUIRE(out_dtype == XB_F32 || out_dtype == XB_F16, XB_ERR_UNSUPPORTED, "xb_shard_combine: output dtype %d", out_dtype);
  if (segments == 0) return 0;
  const size_t esz = out_dtype == XB_F32 ? 4 : 2;
  if (dim % 4 == 0 && out_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(partial) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & (4 * esz - 1)) == 0) {
    const int dim4 = dim / 4;
    const int64_t rows = segments / groups;
    const int64_t blocks4 = std::min<int64_t>((segments * dim4 + 255) / 256, (int64_t)sm_count() * 16);
    const float4* p4 = reinterpret_cast<const float4*>(partial);
    switch (shards) {
      case 2: shard_combine4_kernel<2><<<(unsigned)blocks4, 256, 0, stream>>>(p4, shards, segments, dim4, seg_len, avg, out, out_stride, rows, out_dtype); break;
      case 4: shard_combine4_kernel<4><<<(unsigned)blocks4, 256, 0, stream>>>(p4, shards, segments, dim4, seg_len, avg, out, out_stride, rows, out_dtype); break;
      case 8: shard_combine4_kernel<8><<<(unsigned)blocks4, 256, 0, stream>>>(p4, shards, segments, dim4, seg_len, avg, out, out_stride, rows, out_dtype); break;
      default: shard_combine4_kernel<0><<<(unsigned)blocks4, 256, 0, stream>>>(p4, shards, segments, dim4, seg_len, avg, out, out_stride, rows, out_dtype); break;
    }
    return check_launch("shard_combine4_kernel");
  }
  const int64_t blocks = std::min<int64_t>((segments * dim + 255) / 256, (int64_t)sm_count() * 8);
  shard_combine_kernel<<<(unsigned)blocks, 256, 0, stream>>>(partial, shards, segments, dim, seg_len, avg, out, out_stride, groups,
                                                             out_dtype);
  return check_launch("shard_combine_kernel");
}
