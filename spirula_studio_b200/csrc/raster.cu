// Tile rasteriser, forward and backward (front-to-back alpha blending of the
// depth-sorted splat list of each 16x16 tile).  Restates
// src/kernels/raster/RasterizationEval3DFwd_kernel.cuh:48-313 and
// src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:48-636 (2D variant) with
// the fragment math of src/primitives/Primitive3DGS.cuh:250-300.
//
// Forward: one 128-thread CTA per tile, warp w owning an 8x8 micro-tile and a lane two of its pixels.  The tile's list is
// staged 256 records at a time in shared memory (48-byte gathers); each warp then ballots the staged records against its
// own micro-tile using the record's alpha >= 1/255 ellipse and walks only the records that can touch it, with a warp-wide
// early exit once every lane's transmittance is spent.
//
// Backward: one warp per 8x8 micro-tile.  The warp scans the tile list back to front (starting at the largest
// last-blended index of its pixels), keeps the records whose alpha >= 1/255 ellipse reaches the micro-tile, and works
// through them 32 at a time in two phases: a blend phase with lane = pixel that leaves each (survivor, pixel) fragment in a
// shared-memory matrix, and a reduce phase with lane = survivor that sums its row.  A splat's ten gradient components
// leave as three 16-byte vector reductions per (splat, micro-tile) -- no per-pixel atomics.
#include "ssb_common.cuh"

namespace ssb {

constexpr float kTransmitThreshold = 1e-4f;

__device__ __forceinline__ float eval_alpha(float4 a, float4 b, float px, float py, float& vis, float& sigma, float& dx, float& dy) {
    dx = a.x - px; dy = a.y - py;
    sigma = 0.5f * (b.x * dx * dx + b.z * dy * dy) + b.y * dx * dy;
    vis = __expf(-sigma);
    float alpha = fminf(0.999f, b.w * vis);
    return sigma < 0.f ? 0.f : alpha;
}

// Does the alpha >= 1/255 ellipse of a record reach the box [x0,x1]x[y0,y1]
// (coordinates relative to the splat centre)?  Same construction as the
// reference's micro-tile test (src/core/Common.cuh:55-77), with a small margin
// so rounding can only keep a record, never drop one.
struct EllipseTest { float a, bb2, c, wx, wy; };   // conic scaled to the alpha = 1/255 level set, 2b, and the two tangent slopes

__device__ __forceinline__ EllipseTest ellipse_test_setup(float4 b) {
    // approximate quotients (two units in the last place): the test keeps a margin of 0.01 on a level set at 1
    const float kk = __fdividef(0.5f, __logf(b.w * 255.0f));
    const float a = b.x * kk, c = b.z * kk, bb = b.y * kk;
    EllipseTest t = {a, 2.0f * bb, c, __fdividef(-bb, c), __fdividef(-bb, a)};
    return t;
}

__device__ __forceinline__ bool ellipse_test(const EllipseTest& t, float x0, float x1, float y0, float y1) {
    const float a = t.a, c = t.c, bb = t.bb2;
    const float u0 = fminf(fmaxf(x0 * t.wx, y0), y1), u1 = fminf(fmaxf(x1 * t.wx, y0), y1);
    const float v0 = fminf(fmaxf(y0 * t.wy, x0), x1), v1 = fminf(fmaxf(y1 * t.wy, x0), x1);
    const float mx = fminf(a * x0 * x0 + bb * x0 * u0 + c * u0 * u0, a * x1 * x1 + bb * x1 * u1 + c * u1 * u1);
    const float my = fminf(a * v0 * v0 + bb * v0 * y0 + c * y0 * y0, a * v1 * v1 + bb * v1 * y1 + c * y1 * y1);
    const float mc = fmaxf(fmaxf(x0, -x1), fmaxf(y0, -y1));
    return !(fminf(mc, fminf(mx, my) - 1.0f) >= 0.01f);
}

__device__ __forceinline__ bool ellipse_reaches_box(float4 b, float x0, float x1, float y0, float y1) {
    return ellipse_test(ellipse_test_setup(b), x0, x1, y0, y1);
}

// What bounds a kernel's walk over the sorted list: the entries the list buffer holds, the records the
// record array holds, and where to report an entry that had to be skipped.
struct ListBounds {
    int32_t n_flatten;
    uint32_t n_records;
    unsigned int* status;
};

__device__ __forceinline__ int32_t list_length(const int64_t* __restrict__ n_isects_ptr, const ListBounds& lb) {
    const int64_t m = *n_isects_ptr;
    return (int32_t)(m < 0 ? 0 : (m > lb.n_flatten ? lb.n_flatten : m));
}
__device__ __forceinline__ int32_t clamp_range(int32_t v, int32_t list_len) { return min(max(v, 0), list_len); }
__device__ __forceinline__ bool record_ok(int32_t g, const ListBounds& lb) {
    if ((uint32_t)g < lb.n_records) return true;
    if (lb.status) atomicOr(lb.status, (unsigned int)SSB_STATUS_BAD_INDEX);
    return false;
}

// Forward pass: a CTA of four warps per 16x16 tile, each warp one 8x8 micro-tile, a lane the two pixels (j, i) and
// (j, i + 4).  The tile's list is staged 256 records at a time; every warp keeps the records whose alpha >= 1/255 ellipse
// reaches its micro-tile (in list order) and blends those.  The three shared-memory loads, the list indexing and the loop
// control of a surviving record are spent once for both pixels of a lane, and each lane carries two independent blend
// chains (one pixel per lane with eight warps per tile measured 0.446 ms per 1080p view against 0.396 ms).
constexpr int kFwdThreads = 128;
constexpr int kFwdBatch = 256;

template <bool DEPTH>
__global__ void __launch_bounds__(kFwdThreads) raster_fwd_kernel(
    const SsbScreenRec* __restrict__ screen, const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ flatten_ids,
    const int64_t* __restrict__ n_isects_ptr, ListBounds lb, int I, int W, int H, int tw, int th,
    float* __restrict__ out_rgb, float* __restrict__ out_depth, float* __restrict__ out_T, int32_t* __restrict__ last_ids) {
    __shared__ float4 sA[kFwdBatch], sC[kFwdBatch], sQ[kFwdBatch], sE[kFwdBatch];
    __shared__ float sEw[kFwdBatch];
    __shared__ uint8_t hits[kFwdThreads / 32][kFwdBatch];

    const int img = blockIdx.z;
    const int tile_id = blockIdx.y * tw + blockIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int rx0 = blockIdx.x * kTile + (w & 1) * 8, ry0 = blockIdx.y * kTile + (w >> 1) * 8;
    const int j = rx0 + (lane & 7), i0 = ry0 + (lane >> 3), i1 = i0 + 4;
    const float px = (float)j + 0.5f, py0 = (float)i0 + 0.5f, py1 = (float)i1 + 0.5f;
    const bool in0 = (i0 < H && j < W), in1 = (i1 < H && j < W);
    bool done0 = !in0, done1 = !in1;

    const int32_t* offs = tile_offsets + (int64_t)img * tw * th;
    const int32_t list_len = list_length(n_isects_ptr, lb);
    const int32_t range_start = clamp_range(offs[tile_id], list_len);
    const int32_t range_end = (img == I - 1 && tile_id == tw * th - 1) ? list_len : clamp_range(offs[tile_id + 1], list_len);

    float T0 = 1.0f, T1 = 1.0f;
    float r0 = 0.f, g0 = 0.f, b0 = 0.f, d0 = 0.f, r1 = 0.f, g1 = 0.f, b1 = 0.f, d1 = 0.f;
    int32_t cur0 = 0, cur1 = 0;
    const float fx0 = (float)rx0 + 0.5f, fx1 = (float)rx0 + 7.5f, fy0 = (float)ry0 + 0.5f, fy1 = (float)ry0 + 7.5f;
    const float kLog2e = 1.4426950408889634f;

    for (int32_t batch_start = range_start; batch_start < range_end; batch_start += kFwdBatch) {
        if (__syncthreads_count(done0 && done1) >= kFwdThreads) break;
        const int batch = min(kFwdBatch, range_end - batch_start);
#pragma unroll
        for (int h = 0; h < kFwdBatch / kFwdThreads; ++h) {
            const int e = threadIdx.x + h * kFwdThreads;
            if (e < batch) {
                const int32_t g = flatten_ids[batch_start + e];
                float4 ra = make_float4(-1e30f, -1e30f, 0.f, 0.f), b = make_float4(1.f, 0.f, 1.f, 1.f), rc = make_float4(0.f, 0.f, 0.f, 0.f);
                if (record_ok(g, lb)) {
                    const float4* r = (const float4*)(screen + g);
                    ra = r[0]; b = r[1]; rc = r[2];
                }
                sA[e] = ra; sC[e] = rc;
                sQ[e] = make_float4(0.5f * kLog2e * b.x, kLog2e * b.y, 0.5f * kLog2e * b.z, b.w);
                const EllipseTest et = ellipse_test_setup(b);
                sE[e] = make_float4(et.a, et.bb2, et.c, et.wx);
                sEw[e] = et.wy;
            }
        }
        __syncthreads();
        int n_hit = 0;
        for (int c = 0; c < batch; c += 32) {
            int e = c + lane;
            bool hit = false;
            if (e < batch) {
                float4 a = sA[e];
                hit = (a.x + a.z >= fx0) && (a.x - a.z <= fx1) && (a.y + a.w >= fy0) && (a.y - a.w <= fy1);
                if (hit) {
                    const float4 ev = sE[e];
                    const EllipseTest et = {ev.x, ev.y, ev.z, ev.w, sEw[e]};
                    hit = ellipse_test(et, fx0 - a.x, fx1 - a.x, fy0 - a.y, fy1 - a.y);
                }
            }
            unsigned bal = __ballot_sync(0xffffffffu, hit);
            if (hit) hits[w][n_hit + __popc(bal & ((1u << lane) - 1u))] = (uint8_t)e;
            n_hit += __popc(bal);
        }
        __syncwarp();
#pragma unroll 8
        for (int k = 0; k < n_hit; ++k) {
            if ((k & 7) == 0 && __all_sync(0xffffffffu, done0 && done1)) break;
            const int e = hits[w][k];
            const float4 a = sA[e], b = sQ[e];
            const float dx = a.x - px, dya = a.y - py0, dyb = a.y - py1;
            // q = A dx^2 + dy (B dx + C dy): the two pixels of a lane share dx, so A dx^2 and B dx are formed once
            const float adx2 = b.x * dx * dx, bdx = b.y * dx;
            const float qa = fmaf(dya, fmaf(b.z, dya, bdx), adx2);
            const float qb = fmaf(dyb, fmaf(b.z, dyb, bdx), adx2);
            float va, vb;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(va) : "f"(-qa));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(vb) : "f"(-qb));
            const float alpha_a = fminf(0.999f, b.w * va), alpha_b = fminf(0.999f, b.w * vb);
            const bool ca = !(done0 || !(qa >= 0.f) || alpha_a <= kAlphaThreshold);
            const bool cb = !(done1 || !(qb >= 0.f) || alpha_b <= kAlphaThreshold);
            if (!(ca || cb)) continue;
            const float4 c = sC[e];
            if (ca) {
                const float next_T = T0 * (1.0f - alpha_a);
                if (next_T > kTransmitThreshold) {
                    const float wgt = alpha_a * T0;
                    r0 += c.x * wgt; g0 += c.y * wgt; b0 += c.z * wgt;
                    if (DEPTH) d0 += c.w * wgt;
                    cur0 = batch_start + e;
                    T0 = next_T;
                } else {
                    done0 = true;
                }
            }
            if (cb) {
                const float next_T = T1 * (1.0f - alpha_b);
                if (next_T > kTransmitThreshold) {
                    const float wgt = alpha_b * T1;
                    r1 += c.x * wgt; g1 += c.y * wgt; b1 += c.z * wgt;
                    if (DEPTH) d1 += c.w * wgt;
                    cur1 = batch_start + e;
                    T1 = next_T;
                } else {
                    done1 = true;
                }
            }
        }
    }
    if (in0) {
        const int64_t pix = ((int64_t)img * H + i0) * W + j;
        out_T[pix] = T0;
        out_rgb[3 * pix] = r0; out_rgb[3 * pix + 1] = g0; out_rgb[3 * pix + 2] = b0;
        if (DEPTH) out_depth[pix] = d0 * (1.0f / fmaxf(1.0f - T0, 1e-10f));
        last_ids[pix] = cur0;
    }
    if (in1) {
        const int64_t pix = ((int64_t)img * H + i1) * W + j;
        out_T[pix] = T1;
        out_rgb[3 * pix] = r1; out_rgb[3 * pix + 1] = g1; out_rgb[3 * pix + 2] = b1;
        if (DEPTH) out_depth[pix] = d1 * (1.0f / fmaxf(1.0f - T1, 1e-10f));
        last_ids[pix] = cur1;
    }
}

constexpr int kBwdWarps = 4;          // one 16x16 tile per CTA, one 8x8 micro-tile per warp
constexpr int kBatch = 32;            // survivors per batch: one per lane in the reduction phase
constexpr int kQueue = 96;            // survivor queue (a scan step looks at 64 list entries)
constexpr int kSub = 16;              // survivors per pass through the fragment matrix
constexpr int kMatStride = 64 + 2;    // row stride of the fragment matrix in float2 (64 pixels): rows 16-byte aligned, conflict-free both ways

// What the per-splat densification weight accumulates (DensifyAccumMode, src/primitives/Primitive.cuh:37-39).
struct BwdAccum {
    const float* weight_map;      // [I][H][W] per-pixel weight, or null (all zero)
    const int32_t* gaussian_ids;  // record index -> splat id (packed projection), or null: record index % n_per_image
    int64_t n_per_image;
    float* out;                   // [N]
    float* out_den;               // [N], average mode only
};

// Backward pass.  One warp per 8x8 micro-tile.  The warp walks its tile's list back to front (from the
// largest last-blended index of its pixels), keeps the records whose alpha >= 1/255 ellipse reaches the
// micro-tile, and works through them in batches of 32, each batch in two phases per 8x4 half:
//   blend phase  (lane = pixel): the survivors that reach the half are taken one after another, back to
//                front; every lane evaluates its pixel's alpha, advances its running (T, dL/dT) -- which
//                therefore live in registers -- and leaves the two numbers a fragment's gradients are
//                built from (alpha*T and vis*dL/dalpha) in a 32x32 matrix in shared memory;
//   reduce phase (lane = survivor): every lane sums its survivor's row of the matrix against the pixels'
//                coordinates and colour cotangents: raw moments per pixel row, folded into the micro-tile's
//                moments once per row, and converted to moments about the splat centre at the end.
// The matrix is the transposition between "one lane per pixel", which the blending recurrence wants, and
// "one lane per splat", which lets a splat's gradient leave as three 16-byte reductions per (splat,
// micro-tile) with no cross-lane sums.  All lanes work in both phases; there is no ramp-up or drain.
// ACCUM: 0 none, 1 max, 2 sum, 3 average (sum and denominator) of weight_map[pixel] * alpha * T over the
// fragments a splat contributes (RasterizationEval3DBwd_kernel.cuh:541-550,566-579).
template <bool DEPTH, int ACCUM>
__global__ void __launch_bounds__(kBwdWarps * 32, 4) raster_bwd_kernel(
    const SsbScreenRec* __restrict__ screen, const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ flatten_ids,
    const int64_t* __restrict__ n_isects_ptr, ListBounds lb, int I, int W, int H, int tw, int th,
    const float* __restrict__ render_depth, const float* __restrict__ render_T, const int32_t* __restrict__ last_ids,
    const float* __restrict__ v_rgb, const float* __restrict__ v_depth, const float* __restrict__ v_T,
    SsbScreenRec* __restrict__ v_screen, BwdAccum acc) {
    __shared__ __align__(16) float2 sM[kBwdWarps][kSub * kMatStride];   // [survivor of the pass][pixel]: alpha*T0, vis*dL/dalpha
    __shared__ float4 sSA[kBwdWarps][kBatch];     // survivor: x, y relative to the micro-tile's first pixel centre, list index
    __shared__ float4 sSQ[kBwdWarps][kBatch];     // conic pre-scaled for ex2, opacity
    __shared__ float4 sSC[kBwdWarps][kBatch];     // colour, depth
    __shared__ float4 sV[kBwdWarps][65];          // per pixel: dL/d(rgb), dL/d(depth sum); the lower half sits one entry further (bank offset)
    __shared__ float sW[ACCUM ? kBwdWarps : 1][64];   // weight map of the micro-tile
    __shared__ int32_t sSurv[kBwdWarps][kQueue];  // sorted-list index of each queued survivor
    __shared__ int32_t sSurvG[kBwdWarps][kQueue]; // its record index

    const int img = blockIdx.z;
    const int tile_id = blockIdx.y * tw + blockIdx.x;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int mx0 = blockIdx.x * kTile + (w & 1) * 8, my0 = blockIdx.y * kTile + (w >> 1) * 8;
    if (mx0 >= W || my0 >= H) return;     // whole micro-tile outside the image (warp-uniform)

    const int32_t* offs = tile_offsets + (int64_t)img * tw * th;
    const int32_t list_len = list_length(n_isects_ptr, lb);
    const int32_t range_start = clamp_range(offs[tile_id], list_len);
    const int32_t range_end = (img == I - 1 && tile_id == tw * th - 1) ? list_len : clamp_range(offs[tile_id + 1], list_len);

    // this lane's two pixels: (lane & 7, lane >> 3) in the upper half and four rows below it in the lower one
    const float pxr = (float)(lane & 7), pyr = (float)(lane >> 3);
    float T[2], vT[2], vcx[2], vcy[2], vcz[2], vcw[2];
    int32_t last[2];
    int32_t max_last = -1;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int p = h * 32 + lane;
        const int x = mx0 + (p & 7), y = my0 + (p >> 3);
        const bool inside = x < W && y < H;
        last[h] = -1; T[h] = 0.f; vT[h] = 0.f;
        float4 vc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (inside) {
            const int64_t pix = ((int64_t)img * H + y) * W + x;
            last[h] = last_ids[pix];
            T[h] = render_T[pix];
            vT[h] = v_T ? v_T[pix] : 0.f;
            vc = make_float4(v_rgb[3 * pix], v_rgb[3 * pix + 1], v_rgb[3 * pix + 2], 0.f);
            if (DEPTH) {
                vc.w = v_depth[pix];
                const float inv_alpha = 1.0f / fmaxf(1.0f - T[h], 1e-10f);
                vT[h] += render_depth[pix] * vc.w * inv_alpha;
                vc.w *= inv_alpha;
            }
        }
        if (ACCUM) sW[w][p] = (inside && acc.weight_map) ? acc.weight_map[((int64_t)img * H + y) * W + x] : 0.f;
        vcx[h] = vc.x; vcy[h] = vc.y; vcz[h] = vc.z; vcw[h] = vc.w;
        sV[w][p + h] = vc;
        max_last = max(max_last, last[h]);
    }
    max_last = __reduce_max_sync(0xffffffffu, max_last);
    __syncwarp();

    const float fx0 = (float)mx0 + 0.5f, fx1 = (float)mx0 + 7.5f, fy0 = (float)my0 + 0.5f, fy1 = (float)my0 + 7.5f;
    float2* const M = sM[w];

    int count = 0;                                   // survivors queued
    int32_t pos = min(range_end - 1, max_last);      // top of the 64 list entries looked at next (descending)
    // The walk over the list is two loads deep (list entry -> record), each a trip to L2.  Both are requested
    // ahead of their use: the records of the 64 entries at `pos` while the entries before them are examined,
    // their list entries one step earlier still.  When a batch is full, the records requested last arrive
    // while the batch is worked through.
    int32_t cur_g[2], nxt_g[2];
    float4 cur_a[2], cur_b[2];
    auto load_ids = [&](int32_t top, int32_t (&g)[2]) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int32_t gi = top - (j * 32 + lane);
            g[j] = (top >= range_start && gi >= range_start) ? flatten_ids[gi] : -1;
        }
    };
    auto load_records = [&]() {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            cur_a[j] = make_float4(-1e30f, -1e30f, 0.f, 0.f);      // "reaches nothing"
            cur_b[j] = make_float4(1.f, 0.f, 1.f, 1.f);
            if (cur_g[j] != -1 && record_ok(cur_g[j], lb)) {
                const float4* r = (const float4*)(screen + cur_g[j]);
                cur_a[j] = r[0]; cur_b[j] = r[1];
            }
        }
    };
    load_ids(pos, cur_g);
    load_ids(pos - 64, nxt_g);
    load_records();
    while (true) {
        // ---- queue survivors, back to front, until a full batch is there or the list is used up
        while (pos >= range_start && count < kBatch) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 a = cur_a[j];
                bool ok = (a.x + a.z >= fx0) && (a.x - a.z <= fx1) && (a.y + a.w >= fy0) && (a.y - a.w <= fy1);
                if (ok) ok = ellipse_reaches_box(cur_b[j], fx0 - a.x, fx1 - a.x, fy0 - a.y, fy1 - a.y);
                const unsigned bal = __ballot_sync(0xffffffffu, ok);
                if (ok) {
                    const int slot = count + __popc(bal & ((1u << lane) - 1u));
                    sSurv[w][slot] = pos - (j * 32 + lane);
                    sSurvG[w][slot] = cur_g[j];
                }
                count += __popc(bal);
            }
            pos -= 64;
            cur_g[0] = nxt_g[0]; cur_g[1] = nxt_g[1];
            load_ids(pos - 64, nxt_g);
            load_records();
        }
        if (count == 0) break;
        __syncwarp();
        const int bs = min(kBatch, count);
        // ---- stage the batch: lane l takes survivor l
        const bool active = lane < bs;
        int32_t g = 0;
        float ax = 0.f, ay = 0.f, op = 0.f, cb_a = 0.f, cb_b = 0.f, cb_c = 0.f;
        if (active) {
            const int32_t sidx = sSurv[w][lane];
            g = sSurvG[w][lane];
            const float4* r = (const float4*)(screen + g);
            const float4 a = r[0], b = r[1], c = r[2];
            ax = a.x - fx0; ay = a.y - fy0; op = b.w; cb_a = b.x; cb_b = b.y; cb_c = b.z;
            // conic pre-scaled so that exp(-sigma) = 2^(-q): q = A2 dx^2 + B2 dx dy + C2 dy^2
            const float kLog2e = 1.4426950408889634f;
            sSA[w][lane] = make_float4(ax, ay, __int_as_float(sidx), 0.f);
            sSQ[w][lane] = make_float4(0.5f * kLog2e * b.x, kLog2e * b.y, 0.5f * kLog2e * b.z, b.w);
            sSC[w][lane] = c;
        }
        __syncwarp();
        // raw moments of vis*dL/dalpha over this micro-tile's pixels (coordinates relative to its first pixel centre),
        // and alpha*T0 times the colour cotangent, for the survivor this lane flushes
        float m0 = 0.f, m_x = 0.f, m_y = 0.f, m_xx = 0.f, m_xy = 0.f, m_yy = 0.f, gr = 0.f, gg = 0.f, gb = 0.f, gd = 0.f;
        float aw = 0.f, aw_den = 0.f;
        // two passes of up to 16 survivors through the 16 x 64 fragment matrix
        for (int s0 = 0; s0 < bs; s0 += kSub) {
            const int ns = min(kSub, bs - s0);
            // ---- blend phase: lane = the pixels (lane & 7, lane >> 3) and four rows below it, two independent chains
            {
                float T0a = T[0], vT0a = vT[0], T1a = T[1], vT1a = vT[1];
                const int32_t last0 = last[0], last1 = last[1];
#pragma unroll 4
                for (int k = 0; k < ns; ++k) {
                    const int s = s0 + k;
                    const float4 sa = sSA[w][s];
                    const float4 q4 = sSQ[w][s];
                    const float4 c = sSC[w][s];
                    const float dx = sa.x - pxr;
                    const float adx2 = q4.x * dx * dx, bdx = q4.y * dx;     // shared by the lane's two pixels (same column), as in the forward pass
                    const int32_t sidx = __float_as_int(sa.z);
                    float2 frag[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float dy = sa.y - (pyr + 4.0f * h);
                        const float q = fmaf(dy, fmaf(q4.z, dy, bdx), adx2);
                        float vis;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(vis) : "f"(-q));
                        const float ov = q4.w * vis;
                        const float alpha0 = fminf(0.999f, ov);
                        const bool pass = q >= 0.f && alpha0 > kAlphaThreshold && sidx <= (h ? last1 : last0);
                        // a fragment that does not count is carried through as alpha = 0: it leaves (T, dL/dT) as they are
                        const float alpha = pass ? alpha0 : 0.0f;
                        // a saturated fragment (opacity * vis > 0.999) passes no gradient to its shape
                        const float vis_eff = (pass && ov <= 0.999f) ? vis : 0.0f;
                        const float om = 1.0f - alpha;
                        float& Th = h ? T1a : T0a;
                        float& vTh = h ? vT1a : vT0a;
                        const float Tprev = __fdividef(Th, om);
                        const float cdot = DEPTH ? fmaf(c.x, vcx[h], fmaf(c.y, vcy[h], fmaf(c.z, vcz[h], c.w * vcw[h])))
                                                 : fmaf(c.x, vcx[h], fmaf(c.y, vcy[h], c.z * vcz[h]));
                        const float v_alpha = Tprev * (cdot - vTh);
                        frag[h] = make_float2(alpha * Tprev, vis_eff * v_alpha);
                        vTh = fmaf(alpha, cdot, vTh * om);
                        Th = Tprev;
                    }
                    M[k * kMatStride + lane] = frag[0];
                    M[k * kMatStride + 32 + lane] = frag[1];
                }
                T[0] = T0a; vT[0] = vT0a; T[1] = T1a; vT[1] = vT1a;
            }
            __syncwarp();
            // ---- reduce phase: lane = (survivor lane & 15 of the pass, half lane >> 4): its row of the matrix against the 32 pixels of the half
            {
                const int hh = lane >> 4;
                const float4* row = (const float4*)(M + (lane & 15) * kMatStride + 32 * hh);     // two pixels per 16-byte load
                const float4* vrow = sV[w] + 33 * hh;
                float p0 = 0.f, p_x = 0.f, p_y = 0.f, p_xx = 0.f, p_xy = 0.f, p_yy = 0.f, pr = 0.f, pg = 0.f, pb = 0.f, pd = 0.f, paw = 0.f, paw_den = 0.f;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float r0 = 0.f, r1 = 0.f, r2 = 0.f;        // the row's sums of f, f*x, f*x^2 (f = vis*dL/dalpha)
#pragma unroll
                    for (int xx = 0; xx < 8; xx += 2) {
                        const float4 m = row[(r * 8 + xx) >> 1];          // pixel xx: (m.x, m.y), pixel xx + 1: (m.z, m.w)
                        const float4 vc0 = vrow[r * 8 + xx], vc1 = vrow[r * 8 + xx + 1];
                        r0 += m.y; r1 = fmaf(m.y, (float)xx, r1); r2 = fmaf(m.y, (float)(xx * xx), r2);
                        r0 += m.w; r1 = fmaf(m.w, (float)(xx + 1), r1); r2 = fmaf(m.w, (float)((xx + 1) * (xx + 1)), r2);
                        pr = fmaf(vc0.x, m.x, pr); pg = fmaf(vc0.y, m.x, pg); pb = fmaf(vc0.z, m.x, pb);
                        pr = fmaf(vc1.x, m.z, pr); pg = fmaf(vc1.y, m.z, pg); pb = fmaf(vc1.z, m.z, pb);
                        if (DEPTH) { pd = fmaf(vc0.w, m.x, pd); pd = fmaf(vc1.w, m.z, pd); }
                        if (ACCUM) {
                            const float w0 = sW[w][32 * hh + r * 8 + xx], w1 = sW[w][32 * hh + r * 8 + xx + 1];
                            if (ACCUM == 1) paw = fmaxf(paw, fmaxf(w0 * m.x, w1 * m.z));
                            if (ACCUM >= 2) paw = fmaf(w0, m.x, fmaf(w1, m.z, paw));
                            if (ACCUM == 3) paw_den += m.x + m.z;
                        }
                    }
                    const float yy = (float)(4 * hh + r);
                    p0 += r0; p_x += r1; p_xx += r2;
                    p_y = fmaf(r0, yy, p_y); p_xy = fmaf(r1, yy, p_xy); p_yy = fmaf(r0, yy * yy, p_yy);
                }
                // the two halves of a survivor sit 16 lanes apart: both lanes end up with the micro-tile's sums
                auto both = [](float v) { return v + __shfl_xor_sync(0xffffffffu, v, 16); };
                p0 = both(p0); p_x = both(p_x); p_y = both(p_y); p_xx = both(p_xx); p_xy = both(p_xy); p_yy = both(p_yy);
                pr = both(pr); pg = both(pg); pb = both(pb);
                if (DEPTH) pd = both(pd);
                if (ACCUM == 1) paw = fmaxf(paw, __shfl_xor_sync(0xffffffffu, paw, 16));
                if (ACCUM >= 2) paw = both(paw);
                if (ACCUM == 3) paw_den = both(paw_den);
                // survivor s0 + (lane & 15) is flushed by the lane that staged it: lane s0 + (lane & 15)
                if ((lane >> 4) == (s0 >> 4)) {
                    m0 = p0; m_x = p_x; m_y = p_y; m_xx = p_xx; m_xy = p_xy; m_yy = p_yy; gr = pr; gg = pg; gb = pb; gd = pd; aw = paw; aw_den = paw_den;
                }
            }
            __syncwarp();
        }
        if (active) {
            // moments about the splat centre: sum f*dx = ax*m0 - m_x with dx = ax - x, and so on
            const float s_x = fmaf(ax, m0, -m_x), s_y = fmaf(ay, m0, -m_y);
            const float s_xx = fmaf(ax, fmaf(ax, m0, -2.0f * m_x), m_xx);
            const float s_yy = fmaf(ay, fmaf(ay, m0, -2.0f * m_y), m_yy);
            const float s_xy = fmaf(ax, fmaf(ay, m0, -m_y), fmaf(-ay, m_x, m_xy));
            // dL/dsigma = -opacity * vis * dL/dalpha: the factor common to a splat's fragments is applied here
            const float nx = -op * s_x, ny = -op * s_y;
            const float gca = -0.5f * op * s_xx, gcb = -op * s_xy, gcc = -0.5f * op * s_yy;
            const float gx = cb_a * nx + cb_b * ny, gy = cb_b * nx + cb_c * ny;
            const float gop = m0;
            // non-finite components are dropped, as the reference's atomics do
            // (src/core/Common.cuh:792-856)
            auto fz = [](float v) { return isfinite(v) ? v : 0.0f; };
            float* out = (float*)(v_screen + g);
            if (gx != 0.f || gy != 0.f) red_add_v4(out, fz(gx), fz(gy), 0.f, 0.f);
            if (gca != 0.f || gcb != 0.f || gcc != 0.f || gop != 0.f) red_add_v4(out + 4, fz(gca), fz(gcb), fz(gcc), fz(gop));
            if (gr != 0.f || gg != 0.f || gb != 0.f || gd != 0.f) red_add_v4(out + 8, fz(gr), fz(gg), fz(gb), fz(gd));
            if (ACCUM) {
                const int64_t wid = acc.gaussian_ids ? (int64_t)acc.gaussian_ids[g] : (int64_t)g % acc.n_per_image;
                // weights are products of non-negative factors, so their bit patterns order like integers
                if (ACCUM == 1) { if (aw > 0.f) atomicMax((int*)acc.out + wid, __float_as_int(aw)); }
                else if (aw != 0.f) atomicAdd(acc.out + wid, aw);
                if (ACCUM == 3 && aw_den != 0.f) atomicAdd(acc.out_den + wid, aw_den);
            }
        }
        // ---- the survivors beyond the batch move to the front of the queue
        int32_t keep_i[2] = {0, 0}, keep_g[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (kBatch + j * 32 + lane < count) { keep_i[j] = sSurv[w][kBatch + j * 32 + lane]; keep_g[j] = sSurvG[w][kBatch + j * 32 + lane]; }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (kBatch + j * 32 + lane < count) { sSurv[w][j * 32 + lane] = keep_i[j]; sSurvG[w][j * 32 + lane] = keep_g[j]; }
        count -= bs;
        __syncwarp();
    }
}

static ListBounds make_bounds(int64_t n_records, int64_t n_flatten) {
    ListBounds lb;
    lb.n_flatten = (int32_t)(n_flatten > 0x7fffffff ? 0x7fffffff : n_flatten);
    lb.n_records = (uint32_t)(n_records > 0x7fffffff ? 0x7fffffff : n_records);
    lb.status = device_status_word();
    return lb;
}

static int launch_raster_bwd(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets, const int32_t* d_flatten_ids, int64_t n_flatten, const int64_t* d_n_isects,
                             int32_t n_images, int32_t width, int32_t height, const float* d_render_depth, const float* d_T,
                             const int32_t* d_last_ids, const float* d_v_rgb, const float* d_v_depth, const float* d_v_T,
                             SsbScreenRec* d_v_screen, int accum_mode, BwdAccum acc, void* stream) {
    const int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    const dim3 grid(tw, th, n_images);
    const ListBounds lb = make_bounds(n_records, n_flatten);
#define SSB_RBWD(DEPTH, ACCUM) \
    raster_bwd_kernel<DEPTH, ACCUM><<<grid, kBwdWarps * 32, 0, (cudaStream_t)stream>>>( \
        d_screen, d_tile_offsets, d_flatten_ids, d_n_isects, lb, n_images, width, height, tw, th, d_render_depth, d_T, d_last_ids, d_v_rgb, \
        DEPTH ? d_v_depth : nullptr, d_v_T, d_v_screen, acc)
    // without a depth cotangent the depth channel carries exact zeros: that arithmetic is compiled out
    if (d_v_depth) {
        if (accum_mode == 0) SSB_RBWD(true, 0); else if (accum_mode == 1) SSB_RBWD(true, 1); else if (accum_mode == 2) SSB_RBWD(true, 2); else SSB_RBWD(true, 3);
    } else {
        if (accum_mode == 0) SSB_RBWD(false, 0); else if (accum_mode == 1) SSB_RBWD(false, 1); else if (accum_mode == 2) SSB_RBWD(false, 2); else SSB_RBWD(false, 3);
    }
#undef SSB_RBWD
    SSB_LAUNCHED("raster_bwd_kernel");
    return SSB_OK;
}

}  // namespace ssb

extern "C" {

int ssb_raster_fwd(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                   const int32_t* d_flatten_ids, int64_t n_flatten,
                   const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                   float* d_rgb, float* d_depth, float* d_T, int32_t* d_last_ids, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_screen && d_tile_offsets && d_flatten_ids && d_n_isects && d_rgb && d_T && d_last_ids, "ssb_raster_fwd: NULL argument");
    SSB_REQUIRE(n_images >= 0 && width > 0 && height > 0 && n_records >= 0 && n_flatten >= 0, "ssb_raster_fwd: bad sizes");
    if (n_images == 0) return SSB_OK;
    int tw = (width + kTile - 1) / kTile, th = (height + kTile - 1) / kTile;
    dim3 grid(tw, th, n_images);
    const ListBounds lb = make_bounds(n_records, n_flatten);
    if (d_depth)
        raster_fwd_kernel<true><<<grid, kFwdThreads, 0, (cudaStream_t)stream>>>(d_screen, d_tile_offsets, d_flatten_ids, d_n_isects, lb, n_images, width, height,
                                                                              tw, th, d_rgb, d_depth, d_T, d_last_ids);
    else
        raster_fwd_kernel<false><<<grid, kFwdThreads, 0, (cudaStream_t)stream>>>(d_screen, d_tile_offsets, d_flatten_ids, d_n_isects, lb, n_images, width, height,
                                                                               tw, th, d_rgb, nullptr, d_T, d_last_ids);
    SSB_LAUNCHED("raster_fwd_kernel");
    return SSB_OK;
}

int ssb_raster_bwd(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                   const int32_t* d_flatten_ids, int64_t n_flatten,
                   const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                   const float* d_render_depth, const float* d_T, const int32_t* d_last_ids,
                   const float* d_v_rgb, const float* d_v_depth, const float* d_v_T,
                   SsbScreenRec* d_v_screen, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_screen && d_tile_offsets && d_flatten_ids && d_n_isects && (d_render_depth || !d_v_depth) && d_T && d_last_ids && d_v_rgb && d_v_screen,
                "ssb_raster_bwd: NULL argument");
    SSB_REQUIRE(n_images >= 0 && width > 0 && height > 0 && n_records >= 0 && n_flatten >= 0, "ssb_raster_bwd: bad sizes");
    if (n_images == 0) return SSB_OK;
    return launch_raster_bwd(d_screen, n_records, d_tile_offsets, d_flatten_ids, n_flatten, d_n_isects, n_images, width, height, d_render_depth, d_T, d_last_ids,
                             d_v_rgb, d_v_depth, d_v_T, d_v_screen, 0, BwdAccum{nullptr, nullptr, 1, nullptr, nullptr}, stream);
}

int ssb_raster_bwd_accum(const SsbScreenRec* d_screen, int64_t n_records, const int32_t* d_tile_offsets,
                         const int32_t* d_flatten_ids, int64_t n_flatten,
                         const int64_t* d_n_isects, int32_t n_images, int32_t width, int32_t height,
                         const float* d_render_depth, const float* d_T, const int32_t* d_last_ids,
                         const float* d_v_rgb, const float* d_v_depth, const float* d_v_T, SsbScreenRec* d_v_screen,
                         int32_t accum_mode, const float* d_weight_map, int64_t n_per_image, const int32_t* d_gaussian_ids,
                         float* d_accum_weight, float* d_accum_weight_den, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_screen && d_tile_offsets && d_flatten_ids && d_n_isects && d_T && d_last_ids && d_v_rgb && d_v_screen,
                "ssb_raster_bwd_accum: NULL argument");
    SSB_REQUIRE(n_images >= 0 && width > 0 && height > 0 && n_records >= 0 && n_flatten >= 0, "ssb_raster_bwd_accum: bad sizes");
    SSB_REQUIRE(!d_v_depth || d_render_depth, "ssb_raster_bwd_accum: a depth cotangent needs the rendered depth");
    SSB_REQUIRE(accum_mode >= SSB_ACCUM_NONE && accum_mode <= SSB_ACCUM_AVG, "ssb_raster_bwd_accum: accum_mode %d is not a DensifyAccumMode", accum_mode);
    if (accum_mode != SSB_ACCUM_NONE) {
        SSB_REQUIRE(d_accum_weight, "ssb_raster_bwd_accum: d_accum_weight is NULL");
        SSB_REQUIRE(accum_mode != SSB_ACCUM_AVG || d_accum_weight_den, "ssb_raster_bwd_accum: the average mode needs d_accum_weight_den");
        SSB_REQUIRE(d_gaussian_ids || n_per_image > 0, "ssb_raster_bwd_accum: n_per_image must be positive without d_gaussian_ids");
    }
    if (n_images == 0) return SSB_OK;
    return launch_raster_bwd(d_screen, n_records, d_tile_offsets, d_flatten_ids, n_flatten, d_n_isects, n_images, width, height, d_render_depth, d_T, d_last_ids,
                             d_v_rgb, d_v_depth, d_v_T, d_v_screen, accum_mode,
                             BwdAccum{d_weight_map, d_gaussian_ids, n_per_image > 0 ? n_per_image : 1, d_accum_weight, d_accum_weight_den}, stream);
}

}  // extern "C"
