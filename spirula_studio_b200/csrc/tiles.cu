// Tile intersection: per-pair tile counts, their prefix sum, key generation and
// per-tile ranges.  Restates do_intersect_tile_generic in ellipse mode
// (src/kernels/tile/IntersectTile.cu:34-307,372-509 of the reference).
//
// The integers this stage produces are a function of fp32 arithmetic, so every
// floating-point step is written with round-to-nearest intrinsics (no FMA
// contraction, IEEE division and square root) and the logarithm is a fixed
// polynomial: the same sequence evaluated on any IEEE machine gives the same
// counts, keys and ranges.
//
// The pair count M stays on the device (no host round trip to size the key
// buffers: the caller provides a capacity and later stages read M from memory).
#include "ssb_common.cuh"

namespace ssb {

constexpr int kTilesBlock = 256;
constexpr int kScanItems = 8;                             // per thread
constexpr int kScanChunk = kTilesBlock * kScanItems;      // 2048 counts per block

__device__ __forceinline__ float det_logf(float xin) {
    uint32_t bits = __float_as_uint(xin);
    int e = (int)((bits >> 23) & 255u) - 127;
    float m = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421356f) { m = __fmul_rn(m, 0.5f); e += 1; }
    float f = __fsub_rn(m, 1.0f);
    float z = __fmul_rn(f, f);
    float p = 7.0376836292E-2f;
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.1514610310E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 1.1676998740E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.2420140846E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 1.4249322787E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -1.6668057665E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 2.0000714765E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, -2.4999993993E-1f);
    p = __fmul_rn(p, f); p = __fadd_rn(p, 3.3333331174E-1f);
    float fe = (float)e;
    float y = __fmul_rn(f, z); y = __fmul_rn(y, p);
    float t = __fmul_rn(-2.12194440e-4f, fe); y = __fadd_rn(y, t);
    t = __fmul_rn(0.5f, z); y = __fsub_rn(y, t);
    float r = __fadd_rn(f, y);
    t = __fmul_rn(0.693359375f, fe); r = __fadd_rn(r, t);
    return r;
}

__device__ __forceinline__ float clampf(float x, float a, float b) { return x < a ? a : (x > b ? b : x); }
__device__ __forceinline__ int clampi(int x, int a, int b) { return x < a ? a : (x > b ? b : x); }
// float -> int, NaN -> 0, saturating (cvt.rzi.s32.f32)
__device__ __forceinline__ int f2i(float v) { return __float2int_rz(v); }

__device__ __forceinline__ void ellipse_range_bound(float a, float b, float c, float y0, float y1, float& x0, float& x1) {
    float ac = __fmul_rn(a, c), bb = __fmul_rn(b, b);
    float det = __fsub_rn(ac, bb);
    float q = __fdiv_rn(c, det);
    float sq = __fsqrt_rn(q);
    float nb = -b;
    float r = __fdiv_rn(nb, c);
    float ym = __fmul_rn(r, sq);
    float v0 = clampf(-ym, y0, y1);
    float v1 = clampf(ym, y0, y1);
    float bv0 = __fmul_rn(nb, v0), bv1 = __fmul_rn(nb, v1);
    float inv_a = __fdiv_rn(1.0f, a);
    float t0 = __fmul_rn(c, v0); t0 = __fmul_rn(t0, v0); t0 = __fsub_rn(t0, 1.0f); t0 = __fmul_rn(a, t0);
    float d0 = __fmul_rn(bv0, bv0); d0 = __fsub_rn(d0, t0);
    float t1 = __fmul_rn(c, v1); t1 = __fmul_rn(t1, v1); t1 = __fsub_rn(t1, 1.0f); t1 = __fmul_rn(a, t1);
    float d1 = __fmul_rn(bv1, bv1); d1 = __fsub_rn(d1, t1);
    float e0 = __fsub_rn(bv0, __fsqrt_rn(d0));
    float e1 = __fadd_rn(bv1, __fsqrt_rn(d1));
    x0 = __fmul_rn(inv_a, e0);
    x1 = __fmul_rn(inv_a, e1);
}

struct TileSpan { int xmin, xmax, ymin, ymax; };

template <class F>
__device__ __forceinline__ void for_each_tile(float cx, float cy, float ca, float cb, float cc, const TileSpan& g, F&& fn) {
    const float T = (float)kTile;
    if ((g.ymax - g.ymin) <= (g.xmax - g.xmin)) {
        for (int y = g.ymin; y < g.ymax; ++y) {
            float y0 = __fsub_rn((float)(y * kTile), cy);
            float y1 = __fadd_rn(y0, T);
            float bx0, bx1;
            ellipse_range_bound(ca, cb, cc, y0, y1, bx0, bx1);
            int x0 = f2i(floorf(__fdiv_rn(__fadd_rn(bx0, cx), T)));
            int x1 = f2i(ceilf(__fdiv_rn(__fadd_rn(bx1, cx), T)));
            x0 = clampi(x0, g.xmin, g.xmax);
            x1 = clampi(x1, g.xmin, g.xmax);
            for (int x = x0; x < x1; ++x) fn(x, y);
        }
    } else {
        for (int x = g.xmin; x < g.xmax; ++x) {
            float x0 = __fsub_rn((float)(x * kTile), cx);
            float x1 = __fadd_rn(x0, T);
            float by0, by1;
            ellipse_range_bound(cc, cb, ca, x0, x1, by0, by1);
            int y0 = f2i(floorf(__fdiv_rn(__fadd_rn(by0, cy), T)));
            int y1 = f2i(ceilf(__fdiv_rn(__fadd_rn(by1, cy), T)));
            y0 = clampi(y0, g.ymin, g.ymax);
            y1 = clampi(y1, g.ymin, g.ymax);
            for (int y = y0; y < y1; ++y) fn(x, y);
        }
    }
}

__device__ __forceinline__ bool tile_setup(float4 bb, float4 recb, int tw, int th, TileSpan& g, float conic[3]) {
    if (bb.z <= bb.x || bb.w <= bb.y) return false;
    float ratio = __fdiv_rn(recb.w, kAlphaThreshold);
    float k = __fdiv_rn(0.5f, det_logf(ratio));
    conic[0] = __fmul_rn(recb.x, k); conic[1] = __fmul_rn(recb.y, k); conic[2] = __fmul_rn(recb.z, k);
    const float T = (float)kTile;
    g.xmin = min(max(0, f2i(floorf(__fdiv_rn(__fadd_rn(bb.x, 0.5f), T)))), tw);
    g.ymin = min(max(0, f2i(floorf(__fdiv_rn(__fadd_rn(bb.y, 0.5f), T)))), th);
    g.xmax = min(max(0, f2i(ceilf(__fdiv_rn(__fadd_rn(bb.z, 0.5f), T)))), tw);
    g.ymax = min(max(0, f2i(ceilf(__fdiv_rn(__fadd_rn(bb.w, 0.5f), T)))), th);
    return true;
}

// Pass 1: tiles touched per pair, plus the sum of each 2048-pair chunk.
__global__ void __launch_bounds__(kTilesBlock) tile_count_kernel(
    const float4* __restrict__ aabb, const SsbScreenRec* __restrict__ screen, int64_t total, int tw, int th,
    int32_t* __restrict__ counts, int32_t* __restrict__ chunk_sums) {
    __shared__ int warp_tot[kTilesBlock / 32];
    int64_t base = (int64_t)blockIdx.x * kScanChunk;
    int local = 0;
    for (int it = 0; it < kScanItems; ++it) {
        int64_t idx = base + it * kTilesBlock + threadIdx.x;
        int n = 0;
        if (idx < total) {
            TileSpan g; float cn[3];
            float4 bb = aabb[idx];
            if (bb.z > bb.x && bb.w > bb.y) {
                const float4* r = (const float4*)(screen + idx);
                float4 ra = r[0], rb = r[1];
                if (tile_setup(bb, rb, tw, th, g, cn))
                    for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int, int) { ++n; });
            }
            counts[idx] = n;
        }
        local += n;
    }
    local = __reduce_add_sync(0xffffffffu, local);
    if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int w = 0; w < kTilesBlock / 32; ++w) s += warp_tot[w];
        chunk_sums[blockIdx.x] = s;
    }
}

// Exclusive scan of the chunk sums by one block; also publishes M.
__global__ void __launch_bounds__(1024) chunk_scan_kernel(int32_t* __restrict__ chunk_sums, int n_chunks, int64_t* __restrict__ n_isects) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n_chunks; base += 1024) {
        int i = base + threadIdx.x;
        int64_t v = i < n_chunks ? chunk_sums[i] : 0;
        int64_t inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            int64_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32) {
            int64_t w = warp_tot[threadIdx.x];
            int64_t winc = w;
            for (int o = 1; o < 32; o <<= 1) {
                int64_t t = __shfl_up_sync(0xffffffffu, winc, o);
                if (threadIdx.x >= o) winc += t;
            }
            warp_tot[threadIdx.x] = winc - w;  // exclusive
        }
        __syncthreads();
        int64_t carry = carry_s;
        int64_t excl = carry + warp_tot[threadIdx.x >> 5] + inc - v;
        // chunk sums are stored back as 32-bit offsets; M < 2^31 is enforced by the
        // int32 flatten ids and tile offsets of the interface
        if (i < n_chunks) chunk_sums[i] = (int32_t)excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_isects = carry_s;
}

// Inclusive per-pair prefix within each chunk + chunk offset -> cum_tiles.
__global__ void __launch_bounds__(kTilesBlock) tile_cum_kernel(
    const int32_t* __restrict__ counts, const int32_t* __restrict__ chunk_offsets, int64_t total, int32_t* __restrict__ cum) {
    __shared__ int warp_tot[kTilesBlock / 32];
    __shared__ int carry_s;
    if (threadIdx.x == 0) carry_s = chunk_offsets[blockIdx.x];
    __syncthreads();
    int64_t base = (int64_t)blockIdx.x * kScanChunk;
    for (int it = 0; it < kScanItems; ++it) {
        int64_t idx = base + it * kTilesBlock + threadIdx.x;
        int v = idx < total ? counts[idx] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) woff += warp_tot[w];
        int res = carry_s + woff + inc;
        if (idx < total) cum[idx] = res;
        __syncthreads();
        if (threadIdx.x == kTilesBlock - 1) carry_s = res;
        __syncthreads();
    }
}

// Pass 2: keys and flatten ids.
__global__ void __launch_bounds__(kTilesBlock) tile_emit_kernel(
    const float4* __restrict__ aabb, const float* __restrict__ depths, const SsbScreenRec* __restrict__ screen,
    int64_t total, int64_t n_per_image, int tw, int th, const int32_t* __restrict__ cum, int64_t capacity,
    int64_t* __restrict__ isect_ids, int32_t* __restrict__ flatten_ids) {
    int64_t idx = (int64_t)blockIdx.x * kTilesBlock + threadIdx.x;
    if (idx >= total) return;
    int64_t cur = idx == 0 ? 0 : cum[idx - 1];
    int64_t end = cum[idx];
    if (cur >= end) return;
    if (end > capacity) end = capacity;
    int64_t iid = idx / n_per_image;
    float4 bb = aabb[idx];
    const float4* r = (const float4*)(screen + idx);
    float4 ra = r[0], rb = r[1];
    TileSpan g; float cn[3];
    if (tile_setup(bb, rb, tw, th, g, cn)) {
        uint32_t du = __float_as_uint(fabsf(depths[idx]));
        if (du >> 31) du = ~du; else du ^= (1u << 31);
        int64_t tile_base = iid * tw * th;
        for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int x, int y) {
            if (cur >= end) return;
            int64_t tile_id = tile_base + (int64_t)y * tw + x;
            isect_ids[cur] = (tile_id << 32) | (int64_t)du;
            flatten_ids[cur] = (int32_t)idx;
            ++cur;
        });
    }
    while (cur < end) {
        int64_t tile_id = iid * tw * th;
        isect_ids[cur] = (tile_id << 32) | (int64_t)0xffffffff;
        flatten_ids[cur] = (int32_t)idx;
        ++cur;
    }
}

// offsets[t] = first sorted index whose tile id >= t.
__global__ void tile_ranges_kernel(const int64_t* __restrict__ ids, const int64_t* __restrict__ n_ptr, int64_t capacity,
                                   int64_t n_tiles, int32_t* __restrict__ offsets) {
    int64_t n = min(*n_ptr, capacity);
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n == 0) {
        for (int64_t i = tid; i < n_tiles; i += stride) offsets[i] = 0;
        return;
    }
    for (int64_t idx = tid; idx < n; idx += stride) {
        int64_t tile_id = ids[idx] >> 32;
        if (idx == 0)
            for (int64_t i = 0; i <= tile_id && i < n_tiles; ++i) offsets[i] = 0;
        else {
            int64_t prev = ids[idx - 1] >> 32;
            for (int64_t i = prev + 1; i <= tile_id && i < n_tiles; ++i) offsets[i] = (int32_t)idx;
        }
        if (idx == n - 1)
            for (int64_t i = tile_id + 1; i < n_tiles; ++i) offsets[i] = (int32_t)n;
    }
}

// ---------------------------------------------------------------------------
// Fused intersection: the same sorted lists and ranges without a global sort.
//
// A key is (tile id << 32 | depth bits), so the sorted array is the concatenation of the
// tiles' lists, each ordered by (depth bits, pair index) -- equal keys keep emission order,
// which is pair-index order.  The lists are therefore built directly:
//   1. count the pairs of every tile (one reduction per (splat, tile) pair);
//   2. exclusive scan of the tile counts = the per-tile ranges, and the total M;
//   3. write every pair as (depth bits << 32 | pair index) into its tile's range, at a slot
//      taken from the tile's cursor (arrival order, arbitrary);
//   4. one CTA per tile sorts its range on the whole 64-bit word (all words of a tile are
//      distinct, so the result does not depend on the arrival order) and writes the sorted
//      pair indices and, if asked for, the sorted keys.
// Each pair is written once and read once (8 B) plus its outputs, against five or six
// 24 B/pair passes of the global radix sort.
constexpr int kBinSortThreads = 256;
constexpr int kBinSortCap = 4096;          // longest list sorted in shared memory

__global__ void __launch_bounds__(kTilesBlock) bin_count_kernel(
    const float4* __restrict__ aabb, const SsbScreenRec* __restrict__ screen, int64_t total, int64_t n_per_image, int tw, int th,
    int32_t* __restrict__ tile_count) {
    const int64_t idx = (int64_t)blockIdx.x * kTilesBlock + threadIdx.x;
    if (idx >= total) return;
    const float4 bb = aabb[idx];
    if (!(bb.z > bb.x && bb.w > bb.y)) return;
    const float4* r = (const float4*)(screen + idx);
    const float4 ra = r[0], rb = r[1];
    TileSpan g; float cn[3];
    if (!tile_setup(bb, rb, tw, th, g, cn)) return;
    int32_t* cnt = tile_count + (idx / n_per_image) * tw * th;
    for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int x, int y) { atomicAdd(&cnt[y * tw + x], 1); });
}

// Exclusive scan of the tile counts by one block: offsets[t] (the ranges), the cursors the
// emit pass advances (written over the counts), and M.
__global__ void __launch_bounds__(1024) bin_scan_kernel(int32_t* __restrict__ tile_count, int64_t n_tiles, int32_t* __restrict__ offsets,
                                                        int64_t* __restrict__ n_isects) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int64_t base = 0; base < n_tiles; base += 1024) {
        const int64_t i = base + threadIdx.x;
        const int64_t v = i < n_tiles ? tile_count[i] : 0;
        int64_t inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            int64_t t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32) {
            int64_t w = warp_tot[threadIdx.x];
            int64_t winc = w;
            for (int o = 1; o < 32; o <<= 1) {
                int64_t t = __shfl_up_sync(0xffffffffu, winc, o);
                if (threadIdx.x >= o) winc += t;
            }
            warp_tot[threadIdx.x] = winc - w;
        }
        __syncthreads();
        const int64_t excl = carry_s + warp_tot[threadIdx.x >> 5] + inc - v;
        // positions are 32-bit like the flatten ids and offsets of the interface; ranges past
        // 2^31 - 1 saturate (such a count is far beyond any capacity and is reported as an overflow)
        const int32_t e32 = (int32_t)min(excl, (int64_t)0x7fffffff);
        if (i < n_tiles) { offsets[i] = e32; tile_count[i] = e32; }
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_isects = carry_s;
}

__global__ void __launch_bounds__(kTilesBlock) bin_emit_kernel(
    const float4* __restrict__ aabb, const float* __restrict__ depths, const SsbScreenRec* __restrict__ screen, int64_t total,
    int64_t n_per_image, int tw, int th, int32_t* __restrict__ cursor, int64_t capacity, uint64_t* __restrict__ pairs) {
    const int64_t idx = (int64_t)blockIdx.x * kTilesBlock + threadIdx.x;
    if (idx >= total) return;
    const float4 bb = aabb[idx];
    if (!(bb.z > bb.x && bb.w > bb.y)) return;
    const float4* r = (const float4*)(screen + idx);
    const float4 ra = r[0], rb = r[1];
    TileSpan g; float cn[3];
    if (!tile_setup(bb, rb, tw, th, g, cn)) return;
    uint32_t du = __float_as_uint(fabsf(depths[idx]));
    if (du >> 31) du = ~du; else du ^= (1u << 31);
    const uint64_t word = ((uint64_t)du << 32) | (uint32_t)idx;
    int32_t* cur = cursor + (idx / n_per_image) * tw * th;
    for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int x, int y) {
        const int32_t pos = atomicAdd(&cur[y * tw + x], 1);
        if (pos >= 0 && pos < capacity) pairs[pos] = word;
    });
}

// Sorting network in which every exchange puts the smaller word at the lower index (a bitonic
// merge whose first step mirrors the upper half): positions past the list's end act as
// +infinity without being stored, so any length is sorted in place.
__device__ __forceinline__ void network_sort(uint64_t* a, int n, int padded) {
    for (int lk = 1; (1 << lk) <= padded; ++lk) {
        const int lh = lk - 1, half = 1 << lh;
        for (int t = threadIdx.x; t < (padded >> 1); t += kBinSortThreads) {
            const int blk = t >> lh, off = t & (half - 1);
            const int i = (blk << lk) + off, j = (blk << lk) + (half << 1) - 1 - off;
            if (j < n) { const uint64_t x = a[i], y = a[j]; if (y < x) { a[i] = y; a[j] = x; } }
        }
        __syncthreads();
        for (int ld = lh - 1; ld >= 0; --ld) {
            const int d = 1 << ld;
            for (int t = threadIdx.x; t < (padded >> 1); t += kBinSortThreads) {
                const int i = ((t >> ld) << (ld + 1)) + (t & (d - 1));
                const int j = i + d;
                if (j < n) { const uint64_t x = a[i], y = a[j]; if (y < x) { a[i] = y; a[j] = x; } }
            }
            __syncthreads();
        }
    }
}

__global__ void __launch_bounds__(kBinSortThreads) bin_sort_kernel(
    uint64_t* __restrict__ pairs, const int32_t* __restrict__ offsets, const int64_t* __restrict__ n_isects, int64_t n_tiles,
    int64_t capacity, int64_t* __restrict__ isect_ids, int32_t* __restrict__ flatten_ids) {
    __shared__ uint64_t sm[kBinSortCap];
    const int64_t tile = blockIdx.x;
    const int64_t limit = min(*n_isects, capacity);
    const int64_t start = min((int64_t)offsets[tile], limit);
    const int64_t end = tile + 1 < n_tiles ? min((int64_t)offsets[tile + 1], limit) : limit;
    const int n = (int)(end - start);
    if (n <= 0) return;
    int padded = 1;
    while (padded < n) padded <<= 1;
    uint64_t* seg = pairs + start;
    const uint64_t tile_hi = (uint64_t)tile << 32;
    if (n <= kBinSortCap) {
        for (int i = threadIdx.x; i < n; i += kBinSortThreads) sm[i] = seg[i];
        __syncthreads();
        if (n > 1) network_sort(sm, n, padded);
        for (int i = threadIdx.x; i < n; i += kBinSortThreads) {
            const uint64_t v = sm[i];
            flatten_ids[start + i] = (int32_t)(uint32_t)v;
            if (isect_ids) isect_ids[start + i] = (int64_t)(tile_hi | (v >> 32));
        }
    } else {
        // a list longer than shared memory holds: the same network in place in global memory
        network_sort(seg, n, padded);
        for (int i = threadIdx.x; i < n; i += kBinSortThreads) {
            const uint64_t v = seg[i];
            flatten_ids[start + i] = (int32_t)(uint32_t)v;
            if (isect_ids) isect_ids[start + i] = (int64_t)(tile_hi | (v >> 32));
        }
    }
}

}  // namespace ssb

extern "C" {

int64_t ssb_tile_keys_workspace_bytes(int64_t total) {
    using namespace ssb;
    int64_t chunks = ceil_div(total > 0 ? total : 1, kScanChunk);
    // counts + cum (when the caller passes none) + chunk sums
    return align_up(total * 4, 256) * 2 + align_up(chunks * 4, 256) + 256;
}

int ssb_tile_keys(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                  int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                  void* d_workspace, int64_t workspace_bytes,
                  int32_t* d_tiles_per_splat, int32_t* d_cum_tiles,
                  int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                  int64_t* d_n_isects, int64_t* h_n_isects, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_aabb && d_depths && d_screen && d_workspace && d_isect_ids && d_flatten_ids && d_n_isects, "ssb_tile_keys: NULL argument");
    SSB_REQUIRE(total >= 0 && n_per_image > 0 && width > 0 && height > 0 && capacity >= 0, "ssb_tile_keys: bad sizes");
    SSB_REQUIRE(total < ((int64_t)1 << 31), "ssb_tile_keys: pair index must fit int32");
    SSB_REQUIRE(workspace_bytes >= ssb_tile_keys_workspace_bytes(total), "ssb_tile_keys: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    int64_t chunks = ceil_div(total > 0 ? total : 1, kScanChunk);
    char* ws = (char*)d_workspace;
    int32_t* counts = d_tiles_per_splat ? d_tiles_per_splat : (int32_t*)ws;
    int32_t* cum = d_cum_tiles ? d_cum_tiles : (int32_t*)(ws + align_up(total * 4, 256));
    int32_t* chunk_sums = (int32_t*)(ws + 2 * align_up(total * 4, 256));
    if (total == 0) {
        SSB_CUDA(cudaMemsetAsync(d_n_isects, 0, sizeof(int64_t), st));
    } else {
        tile_count_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>((const float4*)d_aabb, d_screen, total, tw, th, counts, chunk_sums);
        SSB_LAUNCHED("tile_count_kernel");
        chunk_scan_kernel<<<1, 1024, 0, st>>>(chunk_sums, (int)chunks, d_n_isects);
        SSB_LAUNCHED("chunk_scan_kernel");
        tile_cum_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(counts, chunk_sums, total, cum);
        SSB_LAUNCHED("tile_cum_kernel");
        tile_emit_kernel<<<(unsigned)ceil_div(total, kTilesBlock), kTilesBlock, 0, st>>>(
            (const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, cum, capacity, d_isect_ids, d_flatten_ids);
        SSB_LAUNCHED("tile_emit_kernel");
    }
    if (h_n_isects) {
        SSB_CUDA(cudaMemcpyAsync(h_n_isects, d_n_isects, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
        SSB_CUDA(cudaStreamSynchronize(st));
        if (*h_n_isects > capacity) {
            set_error("ssb_tile_keys: %lld (splat, tile) pairs exceed the capacity of %lld", (long long)*h_n_isects, (long long)capacity);
            return SSB_ERR_CAPACITY;
        }
    }
    return SSB_OK;
}

int64_t ssb_intersect_tiles_workspace_bytes(int64_t n_tiles_total, int64_t capacity) {
    using namespace ssb;
    return align_up((n_tiles_total + 1) * 4, 256) + align_up((capacity > 0 ? capacity : 1) * 8, 256);
}

int ssb_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream) {
    return ssb::launch_intersect_tiles(d_aabb, d_depths, d_screen, total, n_per_image, width, height, d_workspace, workspace_bytes,
                                       d_isect_ids, d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream, nullptr);
}

int32_t ssb_tile_n_bits(int64_t n_tiles) {
    int b = 0;
    while (((uint64_t)1 << b) <= (uint64_t)n_tiles) ++b;
    return b;
}

int ssb_tile_ranges(const int64_t* d_sorted_ids, const int64_t* d_n, int64_t capacity, int64_t n_tiles_total, int32_t* d_offsets, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_sorted_ids && d_n && d_offsets && n_tiles_total >= 0 && capacity >= 0, "ssb_tile_ranges: bad argument");
    if (n_tiles_total == 0) return SSB_OK;
    int64_t work = capacity > n_tiles_total ? capacity : n_tiles_total;
    int blocks = (int)(ceil_div(work, 256) < 148 * 8 ? ceil_div(work, 256) : 148 * 8);
    tile_ranges_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(d_sorted_ids, d_n, capacity, n_tiles_total, d_offsets);
    SSB_LAUNCHED("tile_ranges_kernel");
    return SSB_OK;
}

}  // extern "C"

namespace ssb {

// ssb_intersect_tiles with an optional event recorded between the scatter and the per-tile sort
// (the step object times the two halves separately).
int launch_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, cudaEvent_t mark_before_sort) {
    SSB_REQUIRE(d_aabb && d_depths && d_screen && d_workspace && d_flatten_ids && d_tile_offsets && d_n_isects, "ssb_intersect_tiles: NULL argument");
    SSB_REQUIRE(total >= 0 && n_per_image > 0 && width > 0 && height > 0 && capacity >= 0, "ssb_intersect_tiles: bad sizes");
    SSB_REQUIRE(total < ((int64_t)1 << 31) && capacity < ((int64_t)1 << 31), "ssb_intersect_tiles: pair indices and positions must fit int32");
    SSB_REQUIRE(total % n_per_image == 0, "ssb_intersect_tiles: total must be a whole number of images");
    cudaStream_t st = (cudaStream_t)stream;
    const int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    const int64_t n_images = total / n_per_image;
    const int64_t n_tiles = n_images * tw * th;
    SSB_REQUIRE(workspace_bytes >= ssb_intersect_tiles_workspace_bytes(n_tiles, capacity), "ssb_intersect_tiles: workspace too small");
    if (total == 0) {
        SSB_CUDA(cudaMemsetAsync(d_n_isects, 0, sizeof(int64_t), st));
        return SSB_OK;
    }
    SSB_REQUIRE(n_tiles < ((int64_t)1 << 31), "ssb_intersect_tiles: too many tiles");
    char* ws = (char*)d_workspace;
    int32_t* cursor = (int32_t*)ws;
    uint64_t* pairs = (uint64_t*)(ws + align_up((n_tiles + 1) * 4, 256));
    SSB_CUDA(cudaMemsetAsync(cursor, 0, (size_t)n_tiles * 4, st));
    bin_count_kernel<<<(unsigned)ceil_div(total, kTilesBlock), kTilesBlock, 0, st>>>((const float4*)d_aabb, d_screen, total, n_per_image, tw, th, cursor);
    SSB_LAUNCHED("bin_count_kernel");
    bin_scan_kernel<<<1, 1024, 0, st>>>(cursor, n_tiles, d_tile_offsets, d_n_isects);
    SSB_LAUNCHED("bin_scan_kernel");
    bin_emit_kernel<<<(unsigned)ceil_div(total, kTilesBlock), kTilesBlock, 0, st>>>((const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th,
                                                                                    cursor, capacity, pairs);
    SSB_LAUNCHED("bin_emit_kernel");
    if (mark_before_sort) SSB_CUDA(cudaEventRecord(mark_before_sort, st));
    bin_sort_kernel<<<(unsigned)n_tiles, kBinSortThreads, 0, st>>>(pairs, d_tile_offsets, d_n_isects, n_tiles, capacity, d_isect_ids, d_flatten_ids);
    SSB_LAUNCHED("bin_sort_kernel");
    return SSB_OK;
}

}  // namespace ssb
