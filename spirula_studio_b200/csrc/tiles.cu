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

// Tiles touched on one line of a splat's tile rectangle.  A splat is walked along its shorter
// axis (src/kernels/tile/IntersectTile.cu:34-101): by tile rows (row_mode: line = tile y, the
// result is the x span) or by tile columns (line = tile x, the result is the y span).
__device__ __forceinline__ bool tile_row_mode(const TileSpan& g) { return (g.ymax - g.ymin) <= (g.xmax - g.xmin); }

__device__ __forceinline__ void tile_line_span(bool row_mode, int line, float cx, float cy, float ca, float cb, float cc,
                                               const TileSpan& g, int& lo, int& hi) {
    const float T = (float)kTile;
    if (row_mode) {
        float y0 = __fsub_rn((float)(line * kTile), cy);
        float y1 = __fadd_rn(y0, T);
        float bx0, bx1;
        ellipse_range_bound(ca, cb, cc, y0, y1, bx0, bx1);
        int x0 = f2i(floorf(__fdiv_rn(__fadd_rn(bx0, cx), T)));
        int x1 = f2i(ceilf(__fdiv_rn(__fadd_rn(bx1, cx), T)));
        lo = clampi(x0, g.xmin, g.xmax);
        hi = clampi(x1, g.xmin, g.xmax);
    } else {
        float x0 = __fsub_rn((float)(line * kTile), cx);
        float x1 = __fadd_rn(x0, T);
        float by0, by1;
        ellipse_range_bound(cc, cb, ca, x0, x1, by0, by1);
        int y0 = f2i(floorf(__fdiv_rn(__fadd_rn(by0, cy), T)));
        int y1 = f2i(ceilf(__fdiv_rn(__fadd_rn(by1, cy), T)));
        lo = clampi(y0, g.ymin, g.ymax);
        hi = clampi(y1, g.ymin, g.ymax);
    }
}

template <class F>
__device__ __forceinline__ void for_each_tile(float cx, float cy, float ca, float cb, float cc, const TileSpan& g, F&& fn) {
    int lo, hi;
    if (tile_row_mode(g)) {
        for (int y = g.ymin; y < g.ymax; ++y) {
            tile_line_span(true, y, cx, cy, ca, cb, cc, g, lo, hi);
            for (int x = lo; x < hi; ++x) fn(x, y);
        }
    } else {
        for (int x = g.xmin; x < g.xmax; ++x) {
            tile_line_span(false, x, cx, cy, ca, cb, cc, g, lo, hi);
            for (int y = lo; y < hi; ++y) fn(x, y);
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
    const float4* __restrict__ aabb, const SsbScreenRec* __restrict__ screen, int64_t total, int64_t n_per_image, int tw, int th,
    const int32_t* __restrict__ tile_active, int32_t* __restrict__ counts, int32_t* __restrict__ chunk_sums) {
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
                // a tile the live-tile map marks 0 is left out of both passes (src/kernels/tile/IntersectTile.cu:120-122,164-182)
                const int32_t* live = tile_active ? tile_active + (idx / n_per_image) * (int64_t)tw * th : nullptr;
                if (tile_setup(bb, rb, tw, th, g, cn))
                    for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int x, int y) { if (!live || live[y * tw + x]) ++n; });
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
// With a capacity (>= 0): a total beyond it raises SSB_STATUS_PAIRS_DROPPED and, if asked, feeds a running maximum.
__global__ void __launch_bounds__(1024) chunk_scan_kernel(int32_t* __restrict__ chunk_sums, int n_chunks, int64_t* __restrict__ n_isects,
                                                          int64_t capacity = -1, unsigned int* __restrict__ status = nullptr,
                                                          int64_t* __restrict__ running_max = nullptr) {
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
    if (threadIdx.x == 0) {
        const int64_t total = carry_s;
        *n_isects = total;
        if (running_max) atomicMax((long long*)running_max, (long long)total);
        if (capacity >= 0 && total > capacity && status) atomicOr(status, (unsigned int)SSB_STATUS_PAIRS_DROPPED);
    }
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
    int64_t total, int64_t n_per_image, int tw, int th, const int32_t* __restrict__ tile_active, const int32_t* __restrict__ cum,
    int64_t capacity, int64_t* __restrict__ isect_ids, int32_t* __restrict__ flatten_ids) {
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
        const int32_t* live = tile_active ? tile_active + tile_base : nullptr;
        for_each_tile(ra.x, ra.y, cn[0], cn[1], cn[2], g, [&](int x, int y) {
            if (cur >= end) return;
            if (live && !live[y * tw + x]) return;
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

// Live-tile map (tile_active_kernel, src/kernels/tile/IntersectTile.cu:309-344): a tile is live when any pixel of it, grown by
// one pixel on every side and clipped to the image, takes part under the mask [I][Hm][Wm] (nearest-sampled like the loss
// samples it, src/core/Interpolation.cuh:108-120).  One warp per tile: 18 x 18 samples, a ballot per round.
__global__ void __launch_bounds__(256) tile_active_kernel(const uint8_t* __restrict__ mask, int n_images, int Hm, int Wm, int W, int H, int tw, int th,
                                                          int32_t* __restrict__ tile_active) {
    const int64_t t = ((int64_t)blockIdx.x * 256 + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= (int64_t)n_images * tw * th) return;
    const int tx = (int)(t % tw), ty = (int)((t / tw) % th), b = (int)(t / ((int64_t)tw * th));
    constexpr int kEdge = kTile + 2;
    bool live = false;
    for (int base = 0; base < kEdge * kEdge; base += 32) {     // the same number of rounds for every lane
        const int i = base + lane;
        const int y = ty * kTile - 1 + i / kEdge, x = tx * kTile - 1 + i % kEdge;
        if (i < kEdge * kEdge && x >= 0 && y >= 0 && x < W && y < H) {
            const float u = ((float)x + 0.5f) * (float)Wm / (float)W - 0.5f;
            const float v = ((float)y + 0.5f) * (float)Hm / (float)H - 0.5f;
            const int xs = max(0, min(Wm - 1, (int)floorf(u + 0.5f)));
            const int ys = max(0, min(Hm - 1, (int)floorf(v + 0.5f)));
            live |= mask[((int64_t)b * Hm + ys) * Wm + xs] != 0;
        }
        if (__any_sync(0xffffffffu, live)) break;
    }
    live = __any_sync(0xffffffffu, live);
    if (lane == 0) tile_active[t] = live ? 1 : 0;
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
// which is pair-index order.  The lists are built directly, as a two-level bucket sort:
//   0. the range of the depth bits over the visible pairs of each image;
//   1. count the pairs of every bin = (tile, depth bucket): kDepthBuckets buckets per tile, a
//      monotone function of the depth bits (their offset from the image's minimum, shifted so
//      that the image's range fills the buckets), one reduction per (splat, tile) pair;
//   2. exclusive scan of the bin counts = the bins' ranges, every tile's range, and the total M;
//   3. write every pair as (depth bits << 32 | pair index) into its bin, at a slot taken from
//      the bin's cursor (arrival order, arbitrary);
//   4. one CTA per tile orders each of its bins on the whole 64-bit word (all words of a tile are
//      distinct, so the result does not depend on arrival order): a warp ranks a short bin by
//      comparing every word with every other; a long bin goes through a sorting network.
//      The sorted pair indices and, if asked for, the sorted keys are written from there.
// Each pair is written once and read once (8 B) plus its outputs, against five or six
// 24 B/pair passes of the global radix sort.
//
// Passes 1 and 3 walk the splats' tile rectangles line by line.  A thread per splat would leave
// most lanes idle (culled splats, rectangles of different heights), so a warp pools the lines of
// its 32 splats and hands them out one per lane.
constexpr int kBinThreads = 256;
constexpr int kDepthBucketBits = 5;
constexpr int kDepthBuckets = 1 << kDepthBucketBits;
constexpr int kBinSortThreads = 256;
constexpr int kBinSortWarps = kBinSortThreads / 32;
constexpr int kBinSortCap = 4096;          // longest tile list held in shared memory
constexpr int kRankMax = 128;              // longest bin ordered by all-pairs ranking (4 words per lane)
constexpr int64_t kRangeBytes = 4096;      // {min, max} depth words of up to 512 images

__device__ __forceinline__ uint32_t depth_word(float depth) {
    uint32_t du = __float_as_uint(fabsf(depth));
    if (du >> 31) du = ~du; else du ^= (1u << 31);
    return du;
}

// Range of the depth words of each image's visible pairs, kept as {~min, max} so that zeroed
// memory means "none yet" and both ends grow with atomicMax.  A block takes a contiguous span of
// pairs (one image except where two meet), reduces in registers and shared memory and issues two atomics.
__global__ void __launch_bounds__(256) depth_range_kernel(const float4* __restrict__ aabb, const float* __restrict__ depths, int64_t total,
                                                          int64_t n_per_image, uint32_t* __restrict__ range) {
    __shared__ uint32_t s_nlo[8], s_hi[8];
    const int64_t span = (int64_t)gridDim.x * 256;
    const int64_t per_block = (total + span - 1) / span * 256;
    const int64_t begin = (int64_t)blockIdx.x * per_block, end = min(total, begin + per_block);
    if (begin >= end) return;
    const int64_t img_first = begin / n_per_image, img_last = (end - 1) / n_per_image;
    for (int64_t img = img_first; img <= img_last; ++img) {
        const int64_t lo_i = max(begin, img * n_per_image), hi_i = min(end, (img + 1) * n_per_image);
        uint32_t nlo = 0u, hi = 0u;          // ~min and max of what this thread saw
        for (int64_t idx = lo_i + threadIdx.x; idx < hi_i; idx += 256) {
            const float4 bb = aabb[idx];
            if (bb.z > bb.x && bb.w > bb.y) {
                const uint32_t du = depth_word(depths[idx]);
                nlo = max(nlo, ~du); hi = max(hi, du);
            }
        }
        nlo = __reduce_max_sync(0xffffffffu, nlo);
        hi = __reduce_max_sync(0xffffffffu, hi);
        if ((threadIdx.x & 31) == 0) { s_nlo[threadIdx.x >> 5] = nlo; s_hi[threadIdx.x >> 5] = hi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; ++w) { nlo = max(nlo, s_nlo[w]); hi = max(hi, s_hi[w]); }
            if (nlo | hi) { atomicMax(&range[2 * img], nlo); atomicMax(&range[2 * img + 1], hi); }
        }
        __syncthreads();
    }
}

// The same for packed pairs, whose image is looked up per pair and whose count lives on the device.
__global__ void __launch_bounds__(256) depth_range_ids_kernel(const float4* __restrict__ aabb, const float* __restrict__ depths, int64_t max_pairs,
                                                              const int64_t* __restrict__ total_ptr, const int32_t* __restrict__ image_ids,
                                                              uint32_t* __restrict__ range) {
    const int64_t total = min(max_pairs, *total_ptr);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < total; base += stride) {      // warp-uniform trip count
        const int64_t idx = base + threadIdx.x;
        uint32_t nlo = 0u, hi = 0u;
        int img = -1;
        if (idx < total) {
            const float4 bb = aabb[idx];
            if (bb.z > bb.x && bb.w > bb.y) {
                const uint32_t du = depth_word(depths[idx]);
                nlo = ~du; hi = du; img = image_ids[idx];
            }
        }
        // pairs are image-major, so a warp nearly always holds one image
        const int img0 = __reduce_max_sync(0xffffffffu, img);
        if (img0 < 0) continue;
        if (__all_sync(0xffffffffu, img == img0 || img < 0)) {
            nlo = __reduce_max_sync(0xffffffffu, nlo);
            hi = __reduce_max_sync(0xffffffffu, hi);
            if ((threadIdx.x & 31) == 0) { atomicMax(&range[2 * img0], nlo); atomicMax(&range[2 * img0 + 1], hi); }
        } else if (img >= 0) {
            atomicMax(&range[2 * img], nlo); atomicMax(&range[2 * img + 1], hi);
        }
    }
}

__device__ __forceinline__ int depth_bucket(uint32_t du, uint32_t lo, uint32_t hi) {
    const uint32_t span = hi - lo;
    const int used = 32 - __clz(span);                       // bits the offsets occupy (0 when span == 0)
    const int shift = used > kDepthBucketBits ? used - kDepthBucketBits : 0;
    const uint32_t b = (du - lo) >> shift;
    return (int)(b < (uint32_t)kDepthBuckets ? b : (uint32_t)kDepthBuckets - 1u);
}

// Passes 1 (EMIT = false: count) and 3 (EMIT = true: scatter).
// LIVE: tiles whose entry of tile_active [images][th][tw] is 0 take no pairs in either pass.
template <bool EMIT, bool LIVE>
__global__ void __launch_bounds__(kBinThreads) bin_pass_kernel(
    const float4* __restrict__ aabb, const float* __restrict__ depths, const SsbScreenRec* __restrict__ screen, int64_t total,
    int64_t n_per_image, int tw, int th, const uint32_t* __restrict__ range, int32_t* __restrict__ bins, int64_t capacity,
    uint64_t* __restrict__ pairs, const int32_t* __restrict__ image_ids, const int64_t* __restrict__ total_ptr,
    const int32_t* __restrict__ tile_active) {
    // packed input: the image of a pair comes from image_ids and the pair count from device memory
    if (total_ptr) total = min(total, *total_ptr);
    const int lane = threadIdx.x & 31;
    const int64_t idx = (int64_t)blockIdx.x * kBinThreads + threadIdx.x;
    // ---- this lane's splat
    int lines = 0, row_mode = 0;
    TileSpan g = {0, 0, 0, 0};
    float cn[3] = {0.f, 0.f, 0.f}, cx = 0.f, cy = 0.f;
    int32_t bin0 = 0;           // bin of (first tile of the image, this splat's depth bucket)
    uint32_t du = 0;
    if (idx < total) {
        const float4 bb = aabb[idx];
        if (bb.z > bb.x && bb.w > bb.y) {
            const float4* r = (const float4*)(screen + idx);
            const float4 ra = r[0], rb = r[1];
            if (tile_setup(bb, rb, tw, th, g, cn)) {
                cx = ra.x; cy = ra.y;
                row_mode = tile_row_mode(g) ? 1 : 0;
                lines = row_mode ? g.ymax - g.ymin : g.xmax - g.xmin;
                const int64_t img = image_ids ? (int64_t)image_ids[idx] : idx / n_per_image;
                du = depth_word(depths[idx]);
                bin0 = (int32_t)(img * tw * th) * kDepthBuckets + depth_bucket(du, ~range[2 * img], range[2 * img + 1]);
            }
        }
    }
    // ---- pool the warp's lines
    int incl = lines;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
    const int excl = incl - lines;
    const int all = __shfl_sync(0xffffffffu, incl, 31);
    const uint64_t word = ((uint64_t)du << 32) | (uint32_t)idx;
    for (int base = 0; base < all; base += 32) {
        const int item = base + lane;
        // owner = last lane whose first line is <= item (lanes without lines share their successor's start)
        int j = 0;
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) {
            const int cand = j + step;
            const int e = __shfl_sync(0xffffffffu, excl, cand & 31);
            if (cand < 32 && e <= item) j = cand;
        }
        const int o_excl = __shfl_sync(0xffffffffu, excl, j);
        const int o_mode = __shfl_sync(0xffffffffu, row_mode, j);
        TileSpan og;
        og.xmin = __shfl_sync(0xffffffffu, g.xmin, j); og.xmax = __shfl_sync(0xffffffffu, g.xmax, j);
        og.ymin = __shfl_sync(0xffffffffu, g.ymin, j); og.ymax = __shfl_sync(0xffffffffu, g.ymax, j);
        const float ocx = __shfl_sync(0xffffffffu, cx, j), ocy = __shfl_sync(0xffffffffu, cy, j);
        const float oa = __shfl_sync(0xffffffffu, cn[0], j), ob = __shfl_sync(0xffffffffu, cn[1], j), oc = __shfl_sync(0xffffffffu, cn[2], j);
        const int32_t obin = __shfl_sync(0xffffffffu, bin0, j);
        const uint64_t oword = __shfl_sync(0xffffffffu, word, j);
        if (item < all) {
            const int line = (o_mode ? og.ymin : og.xmin) + (item - o_excl);
            int lo, hi;
            tile_line_span(o_mode != 0, line, ocx, ocy, oa, ob, oc, og, lo, hi);
            // tiles of a line are neighbours: along x their bins are kDepthBuckets apart, along y a whole tile row
            int32_t* bin = bins + obin + (o_mode ? line * tw + lo : lo * tw + line) * kDepthBuckets;
            const int step = (o_mode ? 1 : tw) * kDepthBuckets;
            // the bin index / kDepthBuckets is the tile's index over all images, which is how the live-tile map is laid out
            auto is_live = [&](const int32_t* b) { return !LIVE || tile_active[(b - bins) / kDepthBuckets] != 0; };
            if (EMIT) {
                for (int k = lo; k < hi; k += 4) {       // up to four slot requests in flight before the first store
                    int32_t pos[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) pos[u] = (k + u < hi && is_live(bin + u * step)) ? atomicAdd(bin + u * step, 1) : -1;
#pragma unroll
                    for (int u = 0; u < 4; ++u) if (pos[u] >= 0 && pos[u] < capacity) pairs[pos[u]] = oword;
                    bin += 4 * step;
                }
            } else {
                for (int k = lo; k < hi; ++k, bin += step) if (is_live(bin)) atomicAdd(bin, 1);
            }
        }
    }
}

// Exclusive scan of the bin counts, in place, in three launches over 2048-entry chunks.
__global__ void __launch_bounds__(kTilesBlock) bins_chunk_sum_kernel(const int32_t* __restrict__ bins, int64_t n_bins, int32_t* __restrict__ chunk_sums) {
    __shared__ int warp_tot[kTilesBlock / 32];
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    int local = 0;
    for (int it = 0; it < kScanItems; ++it) {
        const int64_t i = base + it * kTilesBlock + threadIdx.x;
        if (i < n_bins) local += bins[i];
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

// bins[i] <- position of bin i's first pair (the cursor the scatter advances);
// offsets[t] <- position of tile t's first pair.
// offsets are clamped to `offset_limit` (the pair capacity): consumers never see a range that leaves the list buffer.
__global__ void __launch_bounds__(kTilesBlock) bins_apply_kernel(int32_t* __restrict__ bins, int64_t n_bins, const int32_t* __restrict__ chunk_offsets,
                                                                 int32_t* __restrict__ offsets, int32_t offset_limit) {
    __shared__ int warp_tot[kTilesBlock / 32];
    __shared__ int carry_s;
    if (threadIdx.x == 0) carry_s = chunk_offsets[blockIdx.x];
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * kScanChunk;
    for (int it = 0; it < kScanItems; ++it) {
        const int64_t i = base + it * kTilesBlock + threadIdx.x;
        const int v = i < n_bins ? bins[i] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) woff += warp_tot[w];
        const int excl = carry_s + woff + inc - v;
        if (i < n_bins) {
            bins[i] = excl;
            if (offsets && (i & (kDepthBuckets - 1)) == 0) offsets[i >> kDepthBucketBits] = min(excl, offset_limit);
        }
        __syncthreads();
        if (threadIdx.x == kTilesBlock - 1) carry_s = excl + v;
        __syncthreads();
    }
}

// Sorting network in which every exchange puts the smaller word at the lower index (a bitonic
// merge whose first step mirrors the upper half): positions past the list's end act as
// +infinity without being stored, so any length is sorted in place.  Whole CTA.
__device__ __forceinline__ void network_sort(uint64_t* a, int n) {
    int padded = 1;
    while (padded < n) padded <<= 1;
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

// A warp orders a bin of at most 32 * E distinct words in place: each lane holds up to E words
// and counts, for each, the words of the bin that are smaller.
template <int E>
__device__ __forceinline__ void rank_sort_warp(uint64_t* a, int n, int lane) {
    uint64_t x[E];
    int rank[E];
#pragma unroll
    for (int e = 0; e < E; ++e) { const int i = e * 32 + lane; x[e] = i < n ? a[i] : ~0ull; rank[e] = 0; }
    for (int t = 0; t < n; ++t) {
        const uint64_t v = a[t];
#pragma unroll
        for (int e = 0; e < E; ++e) rank[e] += v < x[e] ? 1 : 0;
    }
    __syncwarp();
#pragma unroll
    for (int e = 0; e < E; ++e) if (e * 32 + lane < n) a[rank[e]] = x[e];
    __syncwarp();
}

__global__ void __launch_bounds__(kBinSortThreads) bin_sort_kernel(
    uint64_t* __restrict__ pairs, const int32_t* __restrict__ bin_ends, const int64_t* __restrict__ n_isects, int64_t n_tiles,
    int64_t capacity, int64_t* __restrict__ isect_ids, int32_t* __restrict__ flatten_ids) {
    __shared__ uint64_t sm[kBinSortCap];
    __shared__ int edge[kDepthBuckets + 1];       // bin boundaries relative to the tile's first pair
    const int64_t tile = blockIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t limit = min(*n_isects, capacity);
    // after the scatter a bin's cursor stands at its end, which is the next bin's start
    const int64_t first_bin = tile * kDepthBuckets;
    const int64_t start = first_bin == 0 ? 0 : min((int64_t)bin_ends[first_bin - 1], limit);
    if (threadIdx.x <= kDepthBuckets) {
        const int64_t b = first_bin + threadIdx.x - 1;
        edge[threadIdx.x] = (int)((b < 0 ? 0 : min((int64_t)bin_ends[b], limit)) - start);
    }
    __syncthreads();
    const int n = edge[kDepthBuckets];
    if (n <= 0) return;
    uint64_t* seg = pairs + start;
    uint64_t* a = seg;
    if (n <= kBinSortCap) {
        for (int i = threadIdx.x; i < n; i += kBinSortThreads) sm[i] = seg[i];
        a = sm;
        __syncthreads();
    }
    // long bins: the whole CTA, one after another (the loop bounds are the same for every thread)
    for (int b = 0; b < kDepthBuckets; ++b) {
        const int len = edge[b + 1] - edge[b];
        if (len > kRankMax) network_sort(a + edge[b], len);
    }
    // short bins: one warp each
    for (int b = w; b < kDepthBuckets; b += kBinSortWarps) {
        const int len = edge[b + 1] - edge[b];
        if (len <= 1 || len > kRankMax) continue;
        if (len <= 32) rank_sort_warp<1>(a + edge[b], len, lane);
        else if (len <= 64) rank_sort_warp<2>(a + edge[b], len, lane);
        else rank_sort_warp<kRankMax / 32>(a + edge[b], len, lane);
    }
    __syncthreads();
    const uint64_t tile_hi = (uint64_t)tile << 32;
    for (int i = threadIdx.x; i < n; i += kBinSortThreads) {
        const uint64_t v = a[i];
        flatten_ids[start + i] = (int32_t)(uint32_t)v;
        if (isect_ids) isect_ids[start + i] = (int64_t)(tile_hi | (v >> 32));
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

int ssb_tile_keys_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                       int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                       void* d_workspace, int64_t workspace_bytes,
                       int32_t* d_tiles_per_splat, int32_t* d_cum_tiles,
                       int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                       int64_t* d_n_isects, int64_t* h_n_isects, const int32_t* d_tile_active, void* stream) {
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
        tile_count_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>((const float4*)d_aabb, d_screen, total, n_per_image, tw, th, d_tile_active, counts, chunk_sums);
        SSB_LAUNCHED("tile_count_kernel");
        chunk_scan_kernel<<<1, 1024, 0, st>>>(chunk_sums, (int)chunks, d_n_isects, capacity, device_status_word(), nullptr);
        SSB_LAUNCHED("chunk_scan_kernel");
        tile_cum_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(counts, chunk_sums, total, cum);
        SSB_LAUNCHED("tile_cum_kernel");
        tile_emit_kernel<<<(unsigned)ceil_div(total, kTilesBlock), kTilesBlock, 0, st>>>(
            (const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, d_tile_active, cum, capacity, d_isect_ids, d_flatten_ids);
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

int ssb_tile_keys(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                  int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                  void* d_workspace, int64_t workspace_bytes,
                  int32_t* d_tiles_per_splat, int32_t* d_cum_tiles,
                  int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                  int64_t* d_n_isects, int64_t* h_n_isects, void* stream) {
    return ssb_tile_keys_live(d_aabb, d_depths, d_screen, total, n_per_image, width, height, d_workspace, workspace_bytes, d_tiles_per_splat,
                              d_cum_tiles, d_isect_ids, d_flatten_ids, capacity, d_n_isects, h_n_isects, nullptr, stream);
}

int64_t ssb_intersect_tiles_workspace_bytes(int64_t n_tiles_total, int64_t capacity) {
    using namespace ssb;
    const int64_t n_bins = (n_tiles_total > 0 ? n_tiles_total : 1) * kDepthBuckets;
    // bin counters/cursors, chunk sums of their scan, per-image depth range, the unsorted words
    return align_up(n_bins * 4, 256) + align_up(ceil_div(n_bins, kScanChunk) * 4, 256) + kRangeBytes + align_up((capacity > 0 ? capacity : 1) * 8, 256);
}

int ssb_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream) {
    return ssb::launch_intersect_tiles(d_aabb, d_depths, d_screen, total, n_per_image, width, height, d_workspace, workspace_bytes,
                                       d_isect_ids, d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream, nullptr, nullptr, nullptr);
}

int ssb_intersect_tiles_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                             int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                             void* d_workspace, int64_t workspace_bytes,
                             int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                             int32_t* d_tile_offsets, int64_t* d_n_isects, const int32_t* d_tile_active, void* stream) {
    return ssb::launch_intersect_tiles(d_aabb, d_depths, d_screen, total, n_per_image, width, height, d_workspace, workspace_bytes,
                                       d_isect_ids, d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream, nullptr, nullptr, d_tile_active);
}

int ssb_tile_active(const uint8_t* d_mask, int32_t n_images, int32_t mask_h, int32_t mask_w, int32_t width, int32_t height,
                    int32_t* d_tile_active, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_mask && d_tile_active, "ssb_tile_active: NULL argument");
    SSB_REQUIRE(n_images >= 0 && mask_h > 0 && mask_w > 0 && width > 0 && height > 0, "ssb_tile_active: bad sizes");
    const int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    const int64_t n_tiles = (int64_t)n_images * tw * th;
    if (n_tiles == 0) return SSB_OK;
    tile_active_kernel<<<(unsigned)ceil_div(n_tiles * 32, 256), 256, 0, (cudaStream_t)stream>>>(d_mask, n_images, mask_h, mask_w, width, height, tw, th,
                                                                                                d_tile_active);
    SSB_LAUNCHED("tile_active_kernel");
    return SSB_OK;
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
// Packed input (d_image_ids != NULL): `total` is the most pairs there can be, the actual count is read from
// d_total on the device, and n_per_image is ignored in favour of n_images_packed.
static int intersect_tiles_impl(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, cudaEvent_t mark_before_sort,
                        const int32_t* d_image_ids, const int64_t* d_total, int64_t n_images_packed, int64_t* d_max_pairs,
                        const int32_t* d_tile_active);

int launch_intersect_tiles(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, cudaEvent_t mark_before_sort, int64_t* d_max_pairs,
                        const int32_t* d_tile_active) {
    return intersect_tiles_impl(d_aabb, d_depths, d_screen, total, n_per_image, width, height, d_workspace, workspace_bytes, d_isect_ids,
                                d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream, mark_before_sort, nullptr, nullptr, 0, d_max_pairs,
                                d_tile_active);
}

int launch_intersect_tiles_packed(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_image_ids,
                                  const int64_t* d_total, int64_t max_pairs, int64_t n_images, int32_t width, int32_t height,
                                  void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                                  int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, const int32_t* d_tile_active) {
    SSB_REQUIRE(d_image_ids && d_total && n_images > 0, "ssb_intersect_tiles_packed: NULL argument");
    return intersect_tiles_impl(d_aabb, d_depths, d_screen, max_pairs, 1, width, height, d_workspace, workspace_bytes, d_isect_ids,
                                d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream, nullptr, d_image_ids, d_total, n_images, nullptr,
                                d_tile_active);
}

static int intersect_tiles_impl(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen,
                        int64_t total, int64_t n_per_image, int32_t width, int32_t height,
                        void* d_workspace, int64_t workspace_bytes,
                        int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                        int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream, cudaEvent_t mark_before_sort,
                        const int32_t* d_image_ids, const int64_t* d_total, int64_t n_images_packed, int64_t* d_max_pairs,
                        const int32_t* d_tile_active) {
    SSB_REQUIRE(d_aabb && d_depths && d_screen && d_workspace && d_flatten_ids && d_tile_offsets && d_n_isects, "ssb_intersect_tiles: NULL argument");
    SSB_REQUIRE(total >= 0 && n_per_image > 0 && width > 0 && height > 0 && capacity >= 0, "ssb_intersect_tiles: bad sizes");
    SSB_REQUIRE(total < ((int64_t)1 << 31) && capacity < ((int64_t)1 << 31), "ssb_intersect_tiles: pair indices and positions must fit int32");
    SSB_REQUIRE(d_image_ids || total % n_per_image == 0, "ssb_intersect_tiles: total must be a whole number of images");
    cudaStream_t st = (cudaStream_t)stream;
    const int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    const int64_t n_images = d_image_ids ? n_images_packed : total / n_per_image;
    const int64_t n_tiles = n_images * tw * th;
    SSB_REQUIRE(workspace_bytes >= ssb_intersect_tiles_workspace_bytes(n_tiles, capacity), "ssb_intersect_tiles: workspace too small");
    if (total == 0) {
        SSB_CUDA(cudaMemsetAsync(d_n_isects, 0, sizeof(int64_t), st));
        SSB_CUDA(cudaMemsetAsync(d_tile_offsets, 0, (size_t)n_tiles * sizeof(int32_t), st));
        return SSB_OK;
    }
    const int64_t n_bins = n_tiles * kDepthBuckets;
    SSB_REQUIRE(n_bins < ((int64_t)1 << 31), "ssb_intersect_tiles: too many tiles");
    SSB_REQUIRE(n_images * 8 <= kRangeBytes, "ssb_intersect_tiles: at most 512 images per call");
    const int64_t chunks = ceil_div(n_bins, kScanChunk);
    char* ws = (char*)d_workspace;
    uint32_t* range = (uint32_t*)ws;
    int32_t* bins = (int32_t*)(ws + kRangeBytes);
    int32_t* chunk_sums = (int32_t*)((char*)bins + align_up(n_bins * 4, 256));
    uint64_t* pairs = (uint64_t*)((char*)chunk_sums + align_up(chunks * 4, 256));
    SSB_CUDA(cudaMemsetAsync(ws, 0, (size_t)(kRangeBytes + n_bins * 4), st));     // depth ranges and bin counters
    const unsigned range_grid = (unsigned)(ceil_div(total, 256) < 148 * 8 ? ceil_div(total, 256) : 148 * 8);
    if (d_image_ids) depth_range_ids_kernel<<<range_grid, 256, 0, st>>>((const float4*)d_aabb, d_depths, total, d_total, d_image_ids, range);
    else depth_range_kernel<<<range_grid, 256, 0, st>>>((const float4*)d_aabb, d_depths, total, n_per_image, range);
    SSB_LAUNCHED("depth_range_kernel");
    const unsigned pass_grid = (unsigned)ceil_div(total, kBinThreads);
    if (d_tile_active)
        bin_pass_kernel<false, true><<<pass_grid, kBinThreads, 0, st>>>((const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, range, bins, capacity, nullptr, d_image_ids, d_total, d_tile_active);
    else
        bin_pass_kernel<false, false><<<pass_grid, kBinThreads, 0, st>>>((const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, range, bins, capacity, nullptr, d_image_ids, d_total, nullptr);
    SSB_LAUNCHED("bin_pass_kernel<count>");
    bins_chunk_sum_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(bins, n_bins, chunk_sums);
    SSB_LAUNCHED("bins_chunk_sum_kernel");
    chunk_scan_kernel<<<1, 1024, 0, st>>>(chunk_sums, (int)chunks, d_n_isects, capacity, device_status_word(), d_max_pairs);
    SSB_LAUNCHED("chunk_scan_kernel");
    bins_apply_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(bins, n_bins, chunk_sums, d_tile_offsets, (int32_t)capacity);
    SSB_LAUNCHED("bins_apply_kernel");
    if (d_tile_active)
        bin_pass_kernel<true, true><<<pass_grid, kBinThreads, 0, st>>>((const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, range, bins, capacity, pairs, d_image_ids, d_total, d_tile_active);
    else
        bin_pass_kernel<true, false><<<pass_grid, kBinThreads, 0, st>>>((const float4*)d_aabb, d_depths, d_screen, total, n_per_image, tw, th, range, bins, capacity, pairs, d_image_ids, d_total, nullptr);
    SSB_LAUNCHED("bin_pass_kernel<scatter>");
    if (mark_before_sort) SSB_CUDA(cudaEventRecord(mark_before_sort, st));
    bin_sort_kernel<<<(unsigned)n_tiles, kBinSortThreads, 0, st>>>(pairs, bins, d_n_isects, n_tiles, capacity, d_isect_ids, d_flatten_ids);
    SSB_LAUNCHED("bin_sort_kernel");
    return SSB_OK;
}

}  // namespace ssb

// ---------------------------------------------------------------------------
// Packed projection: the visible (view, splat) pairs only, in (view-major, splat-minor) order, with the view
// and splat index of each (projection_3dgs_packed_forward, src/kernels/projection/ProjectionPackedFwd.cu:64-158).
// Like the reference, two passes with a scan between them, and memory proportional to the VISIBLE pairs: the first pass
// evaluates only the cull decision (no SH is read) and leaves one 4-byte flag per pair, the flags are scanned in place,
// and the second pass projects again and writes each kept pair straight to its slot.  The backward pass needs the
// inverse map (pair -> slot), 4 bytes per pair, and then runs the per-splat kernel of the unpacked path: no atomics.
namespace ssb {

__global__ void __launch_bounds__(256) pair_slot_kernel(const int32_t* __restrict__ cam, const int32_t* __restrict__ gid,
                                                        const int64_t* __restrict__ n_pairs, int64_t max_pairs, int64_t n, int64_t total,
                                                        int32_t* __restrict__ pair_of) {
    const int64_t v = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (v >= min(*n_pairs, max_pairs)) return;
    const int64_t i = (int64_t)cam[v] * n + gid[v];
    if (i >= 0 && i < total) pair_of[i] = (int32_t)v;       // ids that name no pair are ignored
}

}  // namespace ssb

extern "C" {

int64_t ssb_project_fwd_packed_workspace_bytes(int64_t n, int32_t n_views) {
    using namespace ssb;
    const int64_t total = (n > 0 ? n : 1) * (n_views > 0 ? n_views : 1);
    return align_up(total * 4, 256) + align_up(ceil_div(total, kScanChunk) * 4, 256);
}

int ssb_project_fwd_packed(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                           void* d_workspace, int64_t workspace_bytes,
                           float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen,
                           int32_t* d_camera_ids, int32_t* d_gaussian_ids, int64_t capacity,
                           int64_t* d_n_visible, int64_t* h_n_visible, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(splats && cams && d_workspace && d_aabb && d_depths && d_screen && d_camera_ids && d_gaussian_ids && d_n_visible,
                "ssb_project_fwd_packed: NULL argument");
    SSB_REQUIRE(n >= 0 && cams->count >= 0 && capacity >= 0, "ssb_project_fwd_packed: bad sizes");
    SSB_REQUIRE(workspace_bytes >= ssb_project_fwd_packed_workspace_bytes(n, cams->count), "ssb_project_fwd_packed: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t total = n * cams->count;
    if (total == 0) {
        SSB_CUDA(cudaMemsetAsync(d_n_visible, 0, sizeof(int64_t), st));
        if (h_n_visible) { SSB_CUDA(cudaStreamSynchronize(st)); *h_n_visible = 0; }
        return SSB_OK;
    }
    char* ws = (char*)d_workspace;
    int32_t* flags = (int32_t*)ws; ws += align_up(total * 4, 256);
    int32_t* chunk_sums = (int32_t*)ws;
    int e = launch_project_fwd_pack_pass(1, splats, shq, n, cams, flags, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, stream);
    if (e) return e;
    const int64_t chunks = ceil_div(total, kScanChunk);
    bins_chunk_sum_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(flags, total, chunk_sums);
    SSB_LAUNCHED("bins_chunk_sum_kernel");
    chunk_scan_kernel<<<1, 1024, 0, st>>>(chunk_sums, (int)chunks, d_n_visible);
    SSB_LAUNCHED("chunk_scan_kernel");
    bins_apply_kernel<<<(unsigned)chunks, kTilesBlock, 0, st>>>(flags, total, chunk_sums, nullptr, 0);
    SSB_LAUNCHED("bins_apply_kernel");
    e = launch_project_fwd_pack_pass(2, splats, shq, n, cams, flags, d_aabb, d_depths, d_radii, d_screen, d_camera_ids, d_gaussian_ids, capacity, stream);
    if (e) return e;
    if (h_n_visible) {
        SSB_CUDA(cudaMemcpyAsync(h_n_visible, d_n_visible, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
        SSB_CUDA(cudaStreamSynchronize(st));
        if (*h_n_visible > capacity) {
            set_error("ssb_project_fwd_packed: %lld visible pairs exceed the capacity of %lld", (long long)*h_n_visible, (long long)capacity);
            return SSB_ERR_CAPACITY;
        }
    }
    return SSB_OK;
}

int64_t ssb_project_bwd_packed_workspace_bytes(int64_t n, int32_t n_views) {
    using namespace ssb;
    const int64_t total = (n > 0 ? n : 1) * (n_views > 0 ? n_views : 1);
    return align_up(total * 4, 256);
}

int ssb_project_bwd_packed(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                           const float* d_aabb, const SsbScreenRec* d_v_screen, const int32_t* d_camera_ids, const int32_t* d_gaussian_ids,
                           const int64_t* d_n_pairs, int64_t max_pairs, void* d_workspace, int64_t workspace_bytes,
                           const SsbSplats* grads, int accumulate, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(splats && cams && d_aabb && d_v_screen && d_camera_ids && d_gaussian_ids && d_n_pairs && d_workspace && grads,
                "ssb_project_bwd_packed: NULL argument");
    SSB_REQUIRE(n >= 0 && max_pairs >= 0, "ssb_project_bwd_packed: bad sizes");
    SSB_REQUIRE((int64_t)cams->count * n < ((int64_t)1 << 31) && max_pairs < ((int64_t)1 << 31), "ssb_project_bwd_packed: pair indices must fit int32");
    SSB_REQUIRE(workspace_bytes >= ssb_project_bwd_packed_workspace_bytes(n, cams->count), "ssb_project_bwd_packed: workspace too small");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t total = n * cams->count;
    if (total == 0) return SSB_OK;
    // slot of every (view, splat) pair in the packed arrays, -1 where the pair was culled; the per-splat kernel of the
    // unpacked path then sums the views of a splat through it, so the result equals the unpacked call's
    int32_t* pair_of = (int32_t*)d_workspace;
    SSB_CUDA(cudaMemsetAsync(pair_of, 0xff, (size_t)total * 4, st));
    if (max_pairs > 0) {
        pair_slot_kernel<<<(unsigned)ceil_div(max_pairs, 256), 256, 0, st>>>(d_camera_ids, d_gaussian_ids, d_n_pairs, max_pairs, n, total, pair_of);
        SSB_LAUNCHED("pair_slot_kernel");
    }
    return launch_project_bwd(splats, shq, n, cams, d_aabb, const_cast<SsbScreenRec*>(d_v_screen), grads, accumulate, 0, stream, pair_of, 0, -1);
}

int ssb_intersect_tiles_packed_live(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_camera_ids,
                                    const int64_t* d_n_pairs, int64_t max_pairs, int32_t n_images, int32_t width, int32_t height,
                                    void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                                    int32_t* d_tile_offsets, int64_t* d_n_isects, const int32_t* d_tile_active, void* stream) {
    return ssb::launch_intersect_tiles_packed(d_aabb, d_depths, d_screen, d_camera_ids, d_n_pairs, max_pairs, n_images, width, height,
                                              d_workspace, workspace_bytes, d_isect_ids, d_flatten_ids, capacity, d_tile_offsets, d_n_isects, stream,
                                              d_tile_active);
}

int ssb_intersect_tiles_packed(const float* d_aabb, const float* d_depths, const SsbScreenRec* d_screen, const int32_t* d_camera_ids,
                               const int64_t* d_n_pairs, int64_t max_pairs, int32_t n_images, int32_t width, int32_t height,
                               void* d_workspace, int64_t workspace_bytes, int64_t* d_isect_ids, int32_t* d_flatten_ids, int64_t capacity,
                               int32_t* d_tile_offsets, int64_t* d_n_isects, void* stream) {
    return ssb_intersect_tiles_packed_live(d_aabb, d_depths, d_screen, d_camera_ids, d_n_pairs, max_pairs, n_images, width, height,
                                           d_workspace, workspace_bytes, d_isect_ids, d_flatten_ids, capacity, d_tile_offsets, d_n_isects, nullptr, stream);
}

}  // extern "C"
