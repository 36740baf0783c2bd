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

}  // extern "C"
