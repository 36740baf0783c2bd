// Per-iteration part of the densification strategy: what engine_densify_step runs on EVERY training step
// (src/engine/EngineDensify.cpp:193-263,355-367), i.e. everything but the periodic relocation.
//
//   ssb_densify_update_scores  one pass over the splats that clips oversized splats (densify_clip_scale_kernel,
//       src/kernels/densify/DensifyScoring.cu:150-178), turns the averaged raster weights into a quotient
//       (densify_accum_finalize_kernel, :281-291) and folds this step's score into the running accumulator
//       (densify_update_weight_kernel, :213-276); then, if asked, the clip of the accumulator at a quantile of its
//       positive entries and the powered copy the sampler reads (densify_clip_score_kernel, :319-343, with the
//       radix-select quantile of src/kernels/densify/Quantile.cu:61-330).
//   ssb_densify_add_noise      the position noise of the MCMC and the revised strategy
//       (mcmc_add_noise_3dgs / revised_add_noise_3dgs, src/shaders/densify.slang:13-74).
//
// The reference issues these as 3 to 12 launches with a gather copy in between; here the per-splat work is one kernel
// and the quantile reads the accumulator in place.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kDensifyThreads = 256;

struct ScoreArgs {
    float max_scale2d, clip_hardness, max_scale3d;
    int finalize_avg, score_mode, weight_by_opacity;
    float blend_w, score_power;
};

// https://www.shadertoy.com/view/4djSRW as the reference spells it (DensifyScoring.cu:200-206)
__device__ __forceinline__ float hash14_fmod(float a, float b, float c, float d) {
    a = fmodf(a * .1031f, 1.0f); b = fmodf(b * .1030f, 1.0f); c = fmodf(c * .0973f, 1.0f); d = fmodf(d * .1099f, 1.0f);
    const float dt = a * (d + 33.33f) + b * (c + 33.33f) + c * (a + 33.33f) + d * (b + 33.33f);
    a += dt; b += dt; c += dt; d += dt;
    return fmodf((a + b) * (c + d), 1.0f);
}

__global__ void __launch_bounds__(kDensifyThreads) densify_score_kernel(
    ScoreArgs a, int64_t n, const float* __restrict__ radii, float* __restrict__ log_scales, const float* __restrict__ logit_opacs,
    float* accum_weight, const float* __restrict__ accum_den, const float* score, const float* __restrict__ score2,
    float* __restrict__ accum_buffer) {
    const int64_t idx = (int64_t)blockIdx.x * kDensifyThreads + threadIdx.x;
    if (idx >= n) return;
    const float radius = radii[idx];
    // ---- oversized splats shrink (screen size) and are capped (world size)
    if (isfinite(a.max_scale2d) || isfinite(a.max_scale3d)) {
        float sx = log_scales[3 * idx], sy = log_scales[3 * idx + 1], sz = log_scales[3 * idx + 2];
        bool touched = false;
        if (isfinite(a.max_scale2d)) {
            float over = radius / a.max_scale2d;
            if (isfinite(a.clip_hardness)) over = fminf(over, a.clip_hardness);
            if (over > 1.0f) {
                const float l = __logf(over);
                sx -= l; sy -= l; sz -= l;
                touched = true;
            }
        }
        if (isfinite(a.max_scale3d)) {
            const float cap = __logf(a.max_scale3d);
            sx = fminf(sx, cap); sy = fminf(sy, cap); sz = fminf(sz, cap);
            touched = true;
        }
        if (touched) { log_scales[3 * idx] = sx; log_scales[3 * idx + 1] = sy; log_scales[3 * idx + 2] = sz; }
    }
    if (!accum_buffer) return;
    // ---- this step's score
    float w;
    if (a.finalize_avg) {                       // [sum(w a T), sum(a T)] -> quotient, kept where the numerator was
        const float den = accum_den[idx];
        const float quot = den > 0.0f ? accum_weight[idx] / den : 0.0f;
        accum_weight[idx] = quot;
        w = score == accum_weight ? quot : score[idx];
    } else {
        w = score[idx];
    }
    if (!(radius > 0.f)) return;
    float weight = fabsf(w);
    if (score2) {                               // geometric blend with the world-gradient score
        weight = powf(weight, 1.0f - a.blend_w) * powf(fabsf(score2[idx]), a.blend_w);
        if (!isfinite(weight)) weight = 0.0f;
    }
    if (a.weight_by_opacity) weight *= 1.0f / (1.0f + __expf(-logit_opacs[idx]));
    if (weight == 0.0f) return;
    if (a.score_power != 1.0f) weight = powf(weight, a.score_power);
    // ---- fold it into the accumulator (x = score, y = steps counted)
    float2 acc = ((float2*)accum_buffer)[idx];
    if (a.score_mode == 1) {                    // Max
        acc.x = fmaxf(acc.x, weight);
        acc.y = fmaxf(acc.y, 1.0f);
    } else if (a.score_mode == 0) {             // Mean
        acc.x = (acc.x * acc.y + weight) / (acc.y + 1.0f);
        acc.y += 1.0f;
    } else if (a.score_mode == 2) {             // Median: a multiplicative random walk toward the sample
        const float r = hash14_fmod(1e2f * weight, 1e2f * acc.x, 1e2f * acc.y, 1e2f * (acc.y + 1.5f));
        if (acc.y == 0.0f) {
            acc.x = weight * exp2f(r - 0.5f);
            acc.y = 1.0f;
        } else {
            acc.x *= exp2f((weight > acc.x ? 1.0f : -1.0f) * r);
            acc.y += 1.0f;
        }
    } else {                                    // Geom
        acc.x = __expf((__logf(fmaxf(acc.x, 1e-30f)) * acc.y + __logf(fmaxf(weight, 1e-30f))) / (acc.y + 1.0f));
        acc.y += 1.0f;
    }
    ((float2*)accum_buffer)[idx] = acc;
}

// ---- quantile of the strictly positive, finite scores, all copies of the maximum left out ------------------------
// Radix select on the float bits, most significant byte first (Quantile.cu:61-330 with one row).  State words:
// [0] max bits, [1] copies of the max, [2] prefix chosen so far, [3] rank still to go, [4] done, [5] result bits,
// [8..263] histogram.
constexpr int kQuantWords = 8 + 256;

__device__ __forceinline__ bool positive_finite(uint32_t u) { return u > 0u && u < 0x7f800000u; }

__global__ void __launch_bounds__(kDensifyThreads) quantile_max_kernel(const float2* __restrict__ acc, int64_t n, uint32_t* __restrict__ st) {
    uint32_t m = 0u;
    for (int64_t i = (int64_t)blockIdx.x * kDensifyThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kDensifyThreads) {
        const uint32_t u = __float_as_uint(acc[i].x);
        if (positive_finite(u)) m = max(m, u);
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0 && m) atomicMax(&st[0], m);
}

__global__ void __launch_bounds__(kDensifyThreads) quantile_hist_kernel(const float2* __restrict__ acc, int64_t n, int pass, uint32_t* __restrict__ st) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t max_copies;
    if (st[4]) return;
    hist[threadIdx.x] = 0u;
    if (threadIdx.x == 0) max_copies = 0u;
    __syncthreads();
    const uint32_t max_bits = st[0], prefix = st[2];
    const uint32_t mask = pass ? 0xFFFFFFFFu << (32 - 8 * pass) : 0u;
    const int shift = 24 - 8 * pass;
    for (int64_t i = (int64_t)blockIdx.x * kDensifyThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kDensifyThreads) {
        const uint32_t u = __float_as_uint(acc[i].x);
        if (!positive_finite(u) || (u & mask) != prefix) continue;
        atomicAdd(&hist[(u >> shift) & 255u], 1u);
        if (pass == 0 && u == max_bits) atomicAdd(&max_copies, 1u);
    }
    __syncthreads();
    if (hist[threadIdx.x]) atomicAdd(&st[8 + threadIdx.x], hist[threadIdx.x]);
    if (pass == 0 && threadIdx.x == 0 && max_copies) atomicAdd(&st[1], max_copies);
}

// One thread: pick the bucket that holds the wanted rank, then clear the histogram for the next pass.
__global__ void quantile_select_kernel(int pass, float q, uint32_t* __restrict__ st) {
    if (!st[4]) {
        const uint32_t max_bits = st[0], max_copies = st[1];
        uint32_t* h = st + 8;
        if (max_bits == 0u) {                   // no positive finite value at all
            st[5] = __float_as_uint(1.0f);
            st[4] = 1u;
        } else {
            bool go = true;
            if (pass == 0) {
                uint64_t total = 0;
                for (int b = 0; b < 256; ++b) total += h[b];
                const uint32_t counted = total > max_copies ? (uint32_t)(total - max_copies) : 0u;
                if (counted == 0u) {            // every value is the maximum
                    st[5] = __float_as_uint(__uint_as_float(max_bits) * 0.5f);
                    st[4] = 1u;
                    go = false;
                } else {
                    st[3] = (uint32_t)(fminf(1.0f, fmaxf(0.0f, q)) * (float)(counted - 1u));     // lower-rank convention
                    st[2] = 0u;
                }
            }
            if (go) {
                uint32_t prefix = st[2], rank = st[3];
                const int shift = 24 - 8 * pass;
                const uint32_t mask = pass ? 0xFFFFFFFFu << (32 - 8 * pass) : 0u;
                const bool drop_max = pass == 0 || (prefix & mask) == (max_bits & mask);
                const uint32_t max_bucket = (max_bits >> shift) & 255u;
                uint32_t cum = 0u, chosen = 255u;
                for (uint32_t b = 0; b < 256u; ++b) {
                    uint32_t c = h[b];
                    if (drop_max && b == max_bucket) c -= max_copies;
                    if (rank < cum + c) { chosen = b; break; }
                    cum += c;
                }
                prefix |= chosen << shift;
                st[2] = prefix;
                st[3] = rank - cum;
                if (pass == 3) { st[5] = prefix; st[4] = 1u; }
            }
        }
    }
    for (int b = 0; b < 256; ++b) st[8 + b] = 0u;
}

__global__ void __launch_bounds__(kDensifyThreads) densify_clip_kernel(int64_t n, float power, float* __restrict__ accum_buffer, const uint32_t* __restrict__ st,
                                                                       float* __restrict__ score_out) {
    const int64_t idx = (int64_t)blockIdx.x * kDensifyThreads + threadIdx.x;
    if (idx >= n) return;
    const float2 a = ((const float2*)accum_buffer)[idx];
    float v = a.x;
    if (st) {
        const float c = __uint_as_float(st[5]);
        if (c > 0.0f && !(v <= c)) {            // also catches NaN
            v = c;
            accum_buffer[2 * idx] = c;
        }
    }
    if (score_out) {
        if (power != 1.0f) v = powf(fmaxf(v, 0.0f), power);
        ((float2*)score_out)[idx] = make_float2(v, a.y);
    }
}

// ---- position noise ------------------------------------------------------------------------------------------------
// Three unit normals from a hash of the splat's own parameters (hash44 + Box-Muller, src/shaders/projection_utils.slang:37-68).
__device__ __forceinline__ float fract_floor(float x) { return x - floorf(x); }

__device__ __forceinline__ float3 randn3_hash(float a, float b, float c, float d) {
    a = fract_floor(a * .1031f); b = fract_floor(b * .1030f); c = fract_floor(c * .0973f); d = fract_floor(d * .1099f);
    const float dt = a * (d + 33.33f) + b * (c + 33.33f) + c * (a + 33.33f) + d * (b + 33.33f);
    a += dt; b += dt; c += dt; d += dt;
    const float hx = fract_floor((a + b) * c), hy = fract_floor((a + c) * b), hz = fract_floor((b + c) * d), hw = fract_floor((c + d) * a);
    const float r0 = sqrtf(-2.0f * logf(1.0f - hx)), r1 = sqrtf(-2.0f * logf(1.0f - hy));
    float s0, c0, c1;
    sincosf(6.28318530718f * hz, &s0, &c0);
    c1 = cosf(6.28318530718f * hw);
    return make_float3(r0 * c0, r0 * s0, r1 * c1);
}

template <bool REVISED>
__global__ void __launch_bounds__(kDensifyThreads) densify_noise_kernel(int64_t n, float scaler, const float* __restrict__ radii, float* __restrict__ means,
                                                                        const float* __restrict__ log_scales, const float* __restrict__ quats,
                                                                        const float* __restrict__ logit_opacs) {
    const int64_t idx = (int64_t)blockIdx.x * kDensifyThreads + threadIdx.x;
    if (idx >= n) return;
    if (REVISED && radii[idx] <= 0.0f) return;          // a splat no view saw stays where it is
    const float mx = means[3 * idx], my = means[3 * idx + 1], mz = means[3 * idx + 2];
    const float lx = log_scales[3 * idx], ly = log_scales[3 * idx + 1], lz = log_scales[3 * idx + 2];
    const float4 q = ((const float4*)quats)[idx];
    const float opac = 1.0f / (1.0f + expf(-logit_opacs[idx]));
    const float3 z = randn3_hash(mx * mx + my * my + mz * mz, mx * lx + my * ly + mz * lz, lx * lx + ly * ly + lz * lz,
                                 (q.x + q.y + q.z + q.w) * opac);
    // rotation of the normalised quaternion (w, x, y, z)
    const float inv = rsqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
    const float w = q.x * inv, x = q.y * inv, y = q.z * inv, zq = q.w * inv;
    const float R[3][3] = {{1.f - 2.f * (y * y + zq * zq), 2.f * (x * y - w * zq), 2.f * (x * zq + w * y)},
                           {2.f * (x * y + w * zq), 1.f - 2.f * (x * x + zq * zq), 2.f * (y * zq - w * x)},
                           {2.f * (x * zq - w * y), 2.f * (y * zq + w * x), 1.f - 2.f * (x * x + y * y)}};
    float s[3], amp;
    if (REVISED) {
        // move along the splat's own axes in proportion to its scale; fade out as it becomes opaque
        s[0] = expf(lx); s[1] = expf(ly); s[2] = expf(lz);
        const float op_pow = powf(1.0f - opac, 150.0f);
        const float extend = sqrtf(2.0f * logf(fmaxf(255.0f * opac, 1.0f)));
        amp = fminf(0.05f * scaler * extend * op_pow, 1.0f);
    } else {
        // covariance-shaped noise, switched off smoothly above opacity 0.005
        s[0] = expf(2.f * lx); s[1] = expf(2.f * ly); s[2] = expf(2.f * lz);
        amp = scaler * (1.0f / (1.0f + expf(-100.0f * ((1.0f - opac) - 0.995f))));
    }
    // R diag(s) R^T (amp z)
    float t[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) t[k] = s[k] * (R[0][k] * z.x + R[1][k] * z.y + R[2][k] * z.z) * amp;
    means[3 * idx] = mx + R[0][0] * t[0] + R[0][1] * t[1] + R[0][2] * t[2];
    means[3 * idx + 1] = my + R[1][0] * t[0] + R[1][1] * t[1] + R[1][2] * t[2];
    means[3 * idx + 2] = mz + R[2][0] * t[0] + R[2][1] * t[1] + R[2][2] * t[2];
}


// ---- periodic part: relocation of dead splats and growth, both by the long-axis split ---------------------------------
// relocate_splats_with_long_axis_split_tensor / add_splats_with_long_axis_split_tensor (src/kernels/densify/Relocation.cu:205-369).
//
// Differences in how, not in what:
//  * the dead splats are listed in ascending order by an ordered compaction (the reference appends them with one atomic
//    per splat, so its order changes from run to run); the number of dead splats stays on the device: the later kernels
//    read it there instead of the host reading it back;
//  * the draw without replacement (Efraimidis-Spirakis keys, smallest k) sorts 64-bit words (key bits, index) with the
//    library's own radix sort; the logarithm in the key is the fixed-operation one, so the draw is the same on every machine.

constexpr int kRelocChunk = 1024;      // splats per block of the ordered compaction

struct DensifyArrays {
    float *means, *quats, *scales, *opacs, *dc, *sh;                 // sh: fp32 values or nullptr
    float *m1[6], *m2[6];                                            // fp32 moments per attribute; [5] = SH or nullptr
    uint8_t* sh_optim_packed; const float4* sh_optim_bounds; int sh_optim_bits;   // 8 / 4, or 0: none
    uint8_t* sh_value_packed; const float2* sh_value_bounds; int sh_value_bits;   // 8 / 16, or 32: none
    float2* accum; int32_t* steps;
};

// bit 0 of flags[i]: the splat stays (it may be drawn from); counts[b]: dead splats of chunk b
__global__ void __launch_bounds__(256) reloc_mask_kernel(int64_t n, float min_opacity, DensifyArrays a, uint8_t* __restrict__ alive,
                                                         int32_t* __restrict__ chunk_dead) {
    __shared__ int warp_cnt[8];
    const int64_t base = (int64_t)blockIdx.x * kRelocChunk;
    int dead = 0;
    for (int k = 0; k < kRelocChunk / 256; ++k) {
        const int64_t i = base + k * 256 + threadIdx.x;
        if (i < n) {
            const float mx = a.means[3 * i], my = a.means[3 * i + 1], mz = a.means[3 * i + 2];
            const float4 q = ((const float4*)a.quats)[i];
            const float sx = a.scales[3 * i], sy = a.scales[3 * i + 1], sz = a.scales[3 * i + 2];
            const float op = a.opacs[i];
            const float cx = a.dc[3 * i], cy = a.dc[3 * i + 1], cz = a.dc[3 * i + 2];
            const bool low = 1.0f / (1.0f + __expf(-op)) <= min_opacity;
            const bool fin = isfinite((mx * mx + my * my + mz * mz) / (q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w) + (sx * cx + sy * cy + sz * cz) * op);
            const bool relocate = low || !fin;
            alive[i] = relocate ? 0 : 1;
            dead += relocate;
        }
    }
    dead = __reduce_add_sync(0xffffffffu, dead);
    if ((threadIdx.x & 31) == 0) warp_cnt[threadIdx.x >> 5] = dead;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < 8; ++w) t += warp_cnt[w];
        chunk_dead[blockIdx.x] = t;
    }
}

// exclusive scan of the chunk counts by one block; total -> *count
__global__ void __launch_bounds__(1024) reloc_scan_kernel(int32_t* __restrict__ chunk_dead, int n_chunks, int32_t* __restrict__ count) {
    __shared__ int warp_tot[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int b0 = 0; b0 < n_chunks; b0 += 1024) {
        const int i = b0 + threadIdx.x;
        const int v = i < n_chunks ? chunk_dead[i] : 0;
        int inc = v;
        for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, inc, o); if ((threadIdx.x & 31) >= o) inc += t; }
        if ((threadIdx.x & 31) == 31) warp_tot[threadIdx.x >> 5] = inc;
        __syncthreads();
        int woff = 0;
        for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) woff += warp_tot[w];
        const int excl = carry + woff + inc - v;
        if (i < n_chunks) chunk_dead[i] = excl;
        __syncthreads();
        if (threadIdx.x == 1023) carry = excl + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) *count = carry;
}

// dead splats written in ascending order: dst[chunk offset + rank inside the chunk]
__global__ void __launch_bounds__(256) reloc_list_kernel(int64_t n, const uint8_t* __restrict__ alive, const int32_t* __restrict__ chunk_off,
                                                         int32_t* __restrict__ dst) {
    __shared__ int warp_cnt[8];
    __shared__ int run;
    if (threadIdx.x == 0) run = chunk_off[blockIdx.x];
    const int64_t base = (int64_t)blockIdx.x * kRelocChunk;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int k = 0; k < kRelocChunk / 256; ++k) {
        const int64_t i = base + k * 256 + threadIdx.x;
        const bool d = i < n && !alive[i];
        const unsigned m = __ballot_sync(0xffffffffu, d);
        if (lane == 0) warp_cnt[w] = __popc(m);
        __syncthreads();
        int off = run;
        for (int x = 0; x < w; ++x) off += warp_cnt[x];
        if (d) dst[off + __popc(m & ((1u << lane) - 1u))] = (int32_t)i;
        __syncthreads();
        if (threadIdx.x == 0) { int t = 0; for (int x = 0; x < 8; ++x) t += warp_cnt[x]; run += t; }
        __syncthreads();
    }
}

__global__ void set_i64_kernel(int64_t* p, int64_t v) { *p = v; }

__device__ __forceinline__ uint32_t hash_u3(uint32_t a, uint32_t b, uint32_t c) {      // src/core/Common.cuh:1019-1039
    uint32_t h = a;
    h *= 0x01000193u; h = (h << 16) | (h >> 16);
    h ^= b; h *= 0x01000193u; h = (h << 16) | (h >> 16);
    h ^= c; h *= 0x01000193u;
    h ^= h >> 15; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}

// Efraimidis-Spirakis: key = w / log(1 - u), u uniform; the k smallest keys are a draw of k without replacement with
// probability proportional to w (compute_efraimidis_spirakis_weight_kernel, DensifySampling.cu:278-296).  The word is
// (order-preserving key bits, index), so a sort on the upper half keeps ties in index order.
__global__ void __launch_bounds__(256) sample_keys_kernel(int64_t n, uint32_t seed, const float2* __restrict__ weights, const uint8_t* __restrict__ alive,
                                                          int64_t* __restrict__ keys, int32_t* __restrict__ vals) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float u = __fmul_rn((float)hash_u3(seed, blockIdx.x, threadIdx.x), 2.3283064365386963e-10f);
    float w = __fdiv_rn(weights[i].x, det_logf(fmaxf(__fsub_rn(1.0f, u), 1e-30f)));
    if (alive && !alive[i]) w = 0.0f;
    if (w == 0.0f) w = 0.0f;                         // -0 and +0 sort together
    uint32_t b = __float_as_uint(w);
    b ^= (b >> 31) ? 0xffffffffu : 0x80000000u;
    keys[i] = (int64_t)(((uint64_t)b << 32) | (uint32_t)i);
    vals[i] = (int32_t)i;
}

__device__ __forceinline__ uint32_t encode_zero(float lo, float hi, float qmax) {      // DensifyQuantCopy.cuh:29-35
    const float range = fmaxf(hi - lo, 1e-30f);
    return (uint32_t)fminf(fmaxf(roundf(qmax * (0.0f - lo) / range), 0.0f), qmax);
}

// One thread per new splat: the source is split along its longest axis into itself and the destination
// (relocate_with_long_axis_split_kernel, Relocation.cu:13-157; long_axis_split_3dgs, src/shaders/densify.slang:76-94).
__global__ void __launch_bounds__(256) reloc_split_kernel(int64_t cur_n, const int32_t* __restrict__ count_ptr, int64_t count_host, float split_k,
                                                          const int32_t* __restrict__ src_idx, const int32_t* __restrict__ dst_idx, DensifyArrays a) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t count = count_ptr ? (int64_t)*count_ptr : count_host;
    if (idx >= count) return;
    const int64_t s = src_idx[idx];
    const int64_t d = dst_idx ? (int64_t)dst_idx[idx] : cur_n + idx;
    // geometry
    const float lx = a.scales[3 * s], ly = a.scales[3 * s + 1], lz = a.scales[3 * s + 2];
    const float4 q = ((const float4*)a.quats)[s];
    const float op = a.opacs[s];
    const float dlen = 0.5f * expf(fmaxf(fmaxf(lx, ly), lz));
    const float kl = -0.6931471805599453f, ks = -0.16251892949777494f;        // log 0.5, log 0.85
    float nx = lx, ny = ly, nz = lz, ex = 0.f, ey = 0.f, ez = 0.f;
    if (lx > ly && lx > lz) { nx += kl; ny += ks; nz += ks; ex = dlen; }
    else if (ly > lz) { nx += ks; ny += kl; nz += ks; ey = dlen; }
    else { nx += ks; ny += ks; nz += kl; ez = dlen; }
    const float inv = rsqrtf(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
    const float w = q.x * inv, x = q.y * inv, y = q.z * inv, z = q.w * inv;
    const float dx = (1.f - 2.f * (y * y + z * z)) * ex + 2.f * (x * y - w * z) * ey + 2.f * (x * z + w * y) * ez;
    const float dy = 2.f * (x * y + w * z) * ex + (1.f - 2.f * (x * x + z * z)) * ey + 2.f * (y * z - w * x) * ez;
    const float dz = 2.f * (x * z - w * y) * ex + 2.f * (y * z + w * x) * ey + (1.f - 2.f * (x * x + y * y)) * ez;
    const float new_op = logf(split_k / (1.0f + expf(-op) - split_k));
    const float mx = a.means[3 * s], my = a.means[3 * s + 1], mz = a.means[3 * s + 2];
    a.means[3 * s] = mx - dx; a.means[3 * s + 1] = my - dy; a.means[3 * s + 2] = mz - dz;
    a.means[3 * d] = mx + dx; a.means[3 * d + 1] = my + dy; a.means[3 * d + 2] = mz + dz;
    a.scales[3 * s] = nx; a.scales[3 * s + 1] = ny; a.scales[3 * s + 2] = nz;
    a.scales[3 * d] = nx; a.scales[3 * d + 1] = ny; a.scales[3 * d + 2] = nz;
    a.opacs[s] = new_op; a.opacs[d] = new_op;
    ((float4*)a.quats)[d] = q;
    // appearance: copied
    for (int k = 0; k < 3; ++k) a.dc[3 * d + k] = a.dc[3 * s + k];
    if (a.sh) for (int k = 0; k < 45; ++k) a.sh[45 * d + k] = a.sh[45 * s + k];
    if (a.sh_value_bits != 32 && a.sh_value_packed) {
        // decode with the source block's bounds, encode against the destination block's CURRENT bounds (clipping is accepted:
        // the next optimiser pass recomputes the bounds; DensifyQuantCopy.cuh:37-77)
        const float qmax = a.sh_value_bits == 16 ? 65535.0f : 255.0f;
        for (int k = 0; k < 45; ++k) {
            const int64_t cs = 45 * s + k, cd = 45 * d + k;
            const float2 ms = a.sh_value_bounds[cs >> 8], md = a.sh_value_bounds[cd >> 8];
            const float code = a.sh_value_bits == 16 ? (float)((const uint16_t*)a.sh_value_packed)[cs] : (float)a.sh_value_packed[cs];
            const float v = ms.x + (ms.y - ms.x) * (code * (1.0f / qmax));
            const float qf = fminf(fmaxf(roundf(qmax * (v - md.x) / fmaxf(md.y - md.x, 1e-30f)), 0.0f), qmax);
            if (a.sh_value_bits == 16) ((uint16_t*)a.sh_value_packed)[cd] = (uint16_t)qf; else a.sh_value_packed[cd] = (uint8_t)qf;
        }
    }
    // optimiser state of the destination: zero (fp32), or the codes that decode nearest to zero against the current bounds
    const int width[6] = {3, 4, 3, 1, 3, 45};
    for (int t = 0; t < 6; ++t)
        if (a.m1[t]) for (int k = 0; k < width[t]; ++k) { a.m1[t][(int64_t)width[t] * d + k] = 0.f; a.m2[t][(int64_t)width[t] * d + k] = 0.f; }
    if (a.sh_optim_bits && a.sh_optim_packed) {
        const float qmax = a.sh_optim_bits == 8 ? 255.0f : 15.0f;
        for (int k = 0; k < 45; ++k) {
            const int64_t c = 45 * d + k;
            const float4 mm = a.sh_optim_bounds[c >> 8];
            const uint32_t uq = encode_zero(mm.x, mm.y, qmax), sq = encode_zero(mm.z, mm.w, qmax);
            if (a.sh_optim_bits == 8) { a.sh_optim_packed[2 * c] = (uint8_t)uq; a.sh_optim_packed[2 * c + 1] = (uint8_t)sq; }
            else a.sh_optim_packed[c] = (uint8_t)((uq & 15u) | ((sq & 15u) << 4));
        }
    }
    if (a.steps) a.steps[d] = 0;
    if (a.accum) a.accum[d] = a.accum[s];
}

}  // namespace ssb

extern "C" {

int64_t ssb_densify_workspace_bytes(int64_t n_splats) {
    (void)n_splats;
    return ssb::kQuantWords * (int64_t)sizeof(uint32_t);
}

int ssb_densify_update_scores(const SsbDensifyScoreConfig* cfg, int64_t n, const float* d_radii, float* d_scales, const float* d_opacities,
                              float* d_accum_weight, const float* d_accum_weight_den, const float* d_world_grad_score, float* d_accum_buffer,
                              float* d_sample_score, void* d_workspace, int64_t workspace_bytes, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(cfg && d_radii && d_scales, "ssb_densify_update_scores: NULL argument");
    SSB_REQUIRE(n >= 0, "ssb_densify_update_scores: bad size");
    SSB_REQUIRE(cfg->score_mode >= 0 && cfg->score_mode <= 3, "ssb_densify_update_scores: score_mode %d is not a DensifyScoreMode", cfg->score_mode);
    SSB_REQUIRE(cfg->accum_mode >= SSB_ACCUM_NONE && cfg->accum_mode <= SSB_ACCUM_AVG, "ssb_densify_update_scores: accum_mode %d is not a DensifyAccumMode",
                cfg->accum_mode);
    SSB_REQUIRE(!d_accum_buffer || d_accum_weight || d_opacities, "ssb_densify_update_scores: no score to fold into the accumulator");
    SSB_REQUIRE(cfg->accum_mode != SSB_ACCUM_AVG || !d_accum_weight || d_accum_weight_den, "ssb_densify_update_scores: d_accum_weight_den is NULL");
    if (n == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    ScoreArgs a;
    a.max_scale2d = cfg->max_screen_size; a.clip_hardness = cfg->max_screen_size_clip_hardness; a.max_scale3d = cfg->max_world_size;
    a.score_mode = cfg->score_mode; a.score_power = cfg->score_power; a.blend_w = cfg->score_blend_world_grad;
    // which buffer is the score (src/engine/EngineDensify.cpp:222-243): the world-gradient score alone at blend 1, else the raster
    // weights with the world-gradient score as blend partner, else the opacities themselves, weighted by the opacity
    const float* score = d_accum_weight;
    const float* score2 = nullptr;
    a.finalize_avg = cfg->accum_mode == SSB_ACCUM_AVG && d_accum_weight != nullptr;
    a.weight_by_opacity = 0;
    if (a.blend_w >= 1.0f && d_world_grad_score) {
        score = d_world_grad_score;              // the averaged weights are still turned into their quotient, as in the reference
    } else if (d_accum_weight) {
        if (a.blend_w > 0.0f && d_world_grad_score) score2 = d_world_grad_score;
    } else {
        score = d_opacities;
        a.weight_by_opacity = 1;
    }
    densify_score_kernel<<<(unsigned)ceil_div(n, kDensifyThreads), kDensifyThreads, 0, st>>>(a, n, d_radii, d_scales, d_opacities, d_accum_weight,
                                                                                          d_accum_weight_den, score, score2, d_accum_buffer);
    SSB_LAUNCHED("densify_score_kernel");
    if (!d_accum_buffer) return SSB_OK;
    const bool clip = cfg->score_clip_quantile > 0.0f && cfg->score_clip_quantile < 1.0f;
    if (!clip && !d_sample_score) return SSB_OK;
    uint32_t* state = nullptr;
    if (clip) {
        SSB_REQUIRE(d_workspace && workspace_bytes >= ssb_densify_workspace_bytes(n), "ssb_densify_update_scores: workspace too small");
        state = (uint32_t*)d_workspace;
        SSB_CUDA(cudaMemsetAsync(state, 0, kQuantWords * sizeof(uint32_t), st));
        const unsigned grid = (unsigned)std::min<int64_t>(ceil_div(n, kDensifyThreads), 148 * 8);
        quantile_max_kernel<<<grid, kDensifyThreads, 0, st>>>((const float2*)d_accum_buffer, n, state);
        SSB_LAUNCHED("quantile_max_kernel");
        for (int pass = 0; pass < 4; ++pass) {
            quantile_hist_kernel<<<grid, kDensifyThreads, 0, st>>>((const float2*)d_accum_buffer, n, pass, state);
            SSB_LAUNCHED("quantile_hist_kernel");
            quantile_select_kernel<<<1, 1, 0, st>>>(pass, cfg->score_clip_quantile, state);
            SSB_LAUNCHED("quantile_select_kernel");
        }
    }
    densify_clip_kernel<<<(unsigned)ceil_div(n, kDensifyThreads), kDensifyThreads, 0, st>>>(n, cfg->final_score_power, d_accum_buffer, state, d_sample_score);
    SSB_LAUNCHED("densify_clip_kernel");
    return SSB_OK;
}

int ssb_densify_add_noise(int64_t n, float scaler, int32_t revised, const float* d_radii, float* d_means, const float* d_scales, const float* d_quats,
                          const float* d_opacities, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_means && d_scales && d_quats && d_opacities && (!revised || d_radii), "ssb_densify_add_noise: NULL argument");
    SSB_REQUIRE(n >= 0, "ssb_densify_add_noise: bad size");
    if (n == 0) return SSB_OK;
    const unsigned grid = (unsigned)ceil_div(n, kDensifyThreads);
    if (revised) densify_noise_kernel<true><<<grid, kDensifyThreads, 0, (cudaStream_t)stream>>>(n, scaler, d_radii, d_means, d_scales, d_quats, d_opacities);
    else densify_noise_kernel<false><<<grid, kDensifyThreads, 0, (cudaStream_t)stream>>>(n, scaler, d_radii, d_means, d_scales, d_quats, d_opacities);
    SSB_LAUNCHED("densify_noise_kernel");
    return SSB_OK;
}


static int densify_arrays(const SsbDensifyState* st, ssb::DensifyArrays* a, const char* who) {
    using namespace ssb;
    SSB_REQUIRE(st, "%s: NULL state", who);
    const SsbSplats& p = st->params;
    SSB_REQUIRE(p.means && p.quats && p.scales && p.opacities && p.features_dc, "%s: parameter arrays missing", who);
    const bool vq = st->sh.d_value_packed && (st->sh.value_bits == 8 || st->sh.value_bits == 16);
    SSB_REQUIRE(vq != (p.features_sh != nullptr), "%s: SH values are either fp32 (params.features_sh) or quantised (sh.d_value_packed)", who);
    SSB_REQUIRE(!vq || st->sh.d_value_bounds, "%s: sh.d_value_bounds is NULL", who);
    const bool oq = st->sh.d_optim_packed != nullptr;
    SSB_REQUIRE(st->sh.layout == SSB_SH_LAYOUT_CELL_BLOCKS, "%s: the SH state must be in the cell-block layout", who);
    SSB_REQUIRE(!oq || (st->sh.d_optim_bounds && (st->sh.optim_bits == 0 || st->sh.optim_bits == 8 || st->sh.optim_bits == 4)), "%s: bad quantised SH state", who);
    *a = DensifyArrays{};
    a->means = p.means; a->quats = p.quats; a->scales = p.scales; a->opacs = p.opacities; a->dc = p.features_dc; a->sh = p.features_sh;
    float* const m1[6] = {st->m1.means, st->m1.quats, st->m1.scales, st->m1.opacities, st->m1.features_dc, oq ? nullptr : st->m1.features_sh};
    float* const m2[6] = {st->m2.means, st->m2.quats, st->m2.scales, st->m2.opacities, st->m2.features_dc, oq ? nullptr : st->m2.features_sh};
    for (int t = 0; t < 6; ++t) {
        SSB_REQUIRE((m1[t] == nullptr) == (m2[t] == nullptr), "%s: first and second moments must come in pairs", who);
        a->m1[t] = m1[t]; a->m2[t] = m2[t];
    }
    a->sh_optim_packed = st->sh.d_optim_packed; a->sh_optim_bounds = (const float4*)st->sh.d_optim_bounds;
    a->sh_optim_bits = oq ? (st->sh.optim_bits ? st->sh.optim_bits : 8) : 0;
    a->sh_value_packed = vq ? (uint8_t*)st->sh.d_value_packed : nullptr; a->sh_value_bounds = (const float2*)st->sh.d_value_bounds;
    a->sh_value_bits = vq ? st->sh.value_bits : 32;
    a->accum = (float2*)st->d_accum_buffer; a->steps = st->d_steps;
    return SSB_OK;
}

// workspace: keys a/b, vals a/b, dead-splat list, alive flags, chunk counts, the count word, the sort's own scratch
struct RelocWs { int64_t *keys_a, *keys_b; int32_t *vals_a, *vals_b, *dst, *chunks, *count; uint8_t* alive; void* sort; int64_t sort_bytes, bytes; };

static RelocWs reloc_ws(void* base, int64_t n) {
    using namespace ssb;
    RelocWs w{};
    int64_t off = 0;
    auto take = [&](int64_t b) { int64_t o = off; off += align_up(b, 256); return base ? (char*)base + o : nullptr; };
    const int64_t m = n > 0 ? n : 1;
    w.keys_a = (int64_t*)take(m * 8); w.keys_b = (int64_t*)take(m * 8);
    w.vals_a = (int32_t*)take(m * 4); w.vals_b = (int32_t*)take(m * 4);
    w.dst = (int32_t*)take(m * 4); w.alive = (uint8_t*)take(m);
    w.chunks = (int32_t*)take(ceil_div(m, kRelocChunk) * 4); w.count = (int32_t*)take(8);
    w.sort_bytes = ssb_sort_workspace_bytes(m);
    w.sort = take(w.sort_bytes);
    w.bytes = off;
    return w;
}

int64_t ssb_densify_relocate_workspace_bytes(int64_t n_splats) { return reloc_ws(nullptr, n_splats).bytes; }

int ssb_densify_relocate(const SsbDensifyState* state, int64_t cur_n, float min_opacity, float split_opacity_k, uint32_t seed, void* d_workspace,
                         int64_t workspace_bytes, int32_t* d_num_relocated, void* stream) {
    using namespace ssb;
    DensifyArrays a;
    if (int e = densify_arrays(state, &a, "ssb_densify_relocate")) return e;
    SSB_REQUIRE(cur_n >= 0 && cur_n < ((int64_t)1 << 30), "ssb_densify_relocate: bad splat count");
    const float* weights = state->d_sample_score ? state->d_sample_score : state->d_accum_buffer;
    SSB_REQUIRE(weights, "ssb_densify_relocate: neither d_sample_score nor d_accum_buffer given");
    SSB_REQUIRE(d_workspace && workspace_bytes >= ssb_densify_relocate_workspace_bytes(cur_n), "ssb_densify_relocate: workspace too small");
    if (cur_n == 0) { if (d_num_relocated) SSB_CUDA(cudaMemsetAsync(d_num_relocated, 0, 4, (cudaStream_t)stream)); return SSB_OK; }
    cudaStream_t st = (cudaStream_t)stream;
    const RelocWs w = reloc_ws(d_workspace, cur_n);
    const int n_chunks = (int)ceil_div(cur_n, kRelocChunk);
    reloc_mask_kernel<<<n_chunks, 256, 0, st>>>(cur_n, min_opacity, a, w.alive, w.chunks);
    SSB_LAUNCHED("reloc_mask_kernel");
    reloc_scan_kernel<<<1, 1024, 0, st>>>(w.chunks, n_chunks, w.count);
    SSB_LAUNCHED("reloc_scan_kernel");
    reloc_list_kernel<<<n_chunks, 256, 0, st>>>(cur_n, w.alive, w.chunks, w.dst);
    SSB_LAUNCHED("reloc_list_kernel");
    if (d_num_relocated) SSB_CUDA(cudaMemcpyAsync(d_num_relocated, w.count, 4, cudaMemcpyDeviceToDevice, st));
    // the draw: every live splat gets a key, the smallest keys win
    sample_keys_kernel<<<(unsigned)ceil_div(cur_n, 256), 256, 0, st>>>(cur_n, seed, (const float2*)weights, w.alive, w.keys_a, w.vals_a);
    SSB_LAUNCHED("sample_keys_kernel");
    int64_t* d_n = (int64_t*)(w.count + 2);       // 8 bytes after the count word, inside its 256-byte slot
    set_i64_kernel<<<1, 1, 0, st>>>(d_n, cur_n);
    SSB_LAUNCHED("set_i64_kernel");
    int32_t sel = 0;
    if (int e = ssb_sort_pairs_u64(w.keys_a, w.vals_a, w.keys_b, w.vals_b, d_n, cur_n, 32, 64, w.sort, w.sort_bytes, &sel, stream)) return e;
    const int32_t* drawn = sel ? w.vals_b : w.vals_a;
    reloc_split_kernel<<<(unsigned)ceil_div(cur_n, 256), 256, 0, st>>>(cur_n, w.count, 0, split_opacity_k, drawn, w.dst, a);
    SSB_LAUNCHED("reloc_split_kernel");
    return SSB_OK;
}

int ssb_densify_add(const SsbDensifyState* state, int64_t cur_n, int64_t num_new, float split_opacity_k, uint32_t seed, void* d_workspace,
                    int64_t workspace_bytes, void* stream) {
    using namespace ssb;
    DensifyArrays a;
    if (int e = densify_arrays(state, &a, "ssb_densify_add")) return e;
    SSB_REQUIRE(cur_n >= 0 && num_new >= 0 && num_new <= cur_n && cur_n + num_new < ((int64_t)1 << 30), "ssb_densify_add: bad counts");
    const float* weights = state->d_sample_score ? state->d_sample_score : state->d_accum_buffer;
    SSB_REQUIRE(weights, "ssb_densify_add: neither d_sample_score nor d_accum_buffer given");
    SSB_REQUIRE(d_workspace && workspace_bytes >= ssb_densify_relocate_workspace_bytes(cur_n), "ssb_densify_add: workspace too small");
    if (num_new == 0) return SSB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const RelocWs w = reloc_ws(d_workspace, cur_n);
    sample_keys_kernel<<<(unsigned)ceil_div(cur_n, 256), 256, 0, st>>>(cur_n, seed, (const float2*)weights, nullptr, w.keys_a, w.vals_a);
    SSB_LAUNCHED("sample_keys_kernel");
    int64_t* d_n = (int64_t*)(w.count + 2);
    set_i64_kernel<<<1, 1, 0, st>>>(d_n, cur_n);
    SSB_LAUNCHED("set_i64_kernel");
    int32_t sel = 0;
    if (int e = ssb_sort_pairs_u64(w.keys_a, w.vals_a, w.keys_b, w.vals_b, d_n, cur_n, 32, 64, w.sort, w.sort_bytes, &sel, stream)) return e;
    const int32_t* drawn = sel ? w.vals_b : w.vals_a;
    reloc_split_kernel<<<(unsigned)ceil_div(num_new, 256), 256, 0, st>>>(cur_n, nullptr, num_new, split_opacity_k, drawn, nullptr, a);
    SSB_LAUNCHED("reloc_split_kernel");
    return SSB_OK;
}

}  // extern "C"
