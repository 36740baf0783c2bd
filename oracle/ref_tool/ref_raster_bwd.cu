// TEST INFRASTRUCTURE.  The reference's tile rasteriser backward kernel, 2D variant
// (src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:48-744 via
// RasterizationBwd_kernel.cuh) for Vanilla3DGS<3>, launched on raw device buffers.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/raster/RasterizationBwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

extern "C" int ref_raster_bwd(
    uint32_t I, uint32_t N, uint32_t n_isects, uint32_t W, uint32_t H,
    float* xy, float* depth, float* conic, float* opac, float* rgb,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* render_rgb, float* render_depth, const float* render_T, const int32_t* last_ids,
    float* v_render_rgb, float* v_render_depth, const float* v_render_T,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb) {
    RawScreen screen((int64_t)I * N, xy, depth, conic, opac, rgb);
    RawScreen v_screen((int64_t)I * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
    RefPrim::WorldBuffer world, v_world;
    RenderOutput::Buffer out, dist, v_out, v_dist;
    out.rgbs = (float3*)render_rgb; out.depths = render_depth;
    v_out.rgbs = (float3*)v_render_rgb; v_out.depths = v_render_depth;
    uint32_t tw = (W + 15) / 16, th = (H + 15) / 16;
    rasterize_to_pixels_bwd_kernel_wrapper<RefPrim, DistortionType::None, DensifyAccumMode::None, false>(
        0, I, N, n_isects, nullptr, world, screen, W, H, tw, th, tile_offsets, flatten_ids,
        render_T, last_ids, out, dist, nullptr, nullptr, v_out, v_render_T, nullptr, v_dist,
        v_world, v_screen, nullptr, nullptr);
    return ref_finish();
}

// The same launch with a densification weight map: mode 1 = Max, 2 = Sum, 3 = Avg (DensifyAccumMode,
// src/primitives/Primitive.cuh:37-39); o_accum_weight [N] (and o_accum_weight_den [N] for Avg) zeroed by the caller.
extern "C" int ref_raster_bwd_accum(
    int mode, uint32_t I, uint32_t N, uint32_t n_isects, uint32_t W, uint32_t H,
    float* xy, float* depth, float* conic, float* opac, float* rgb,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* render_rgb, float* render_depth, const float* render_T, const int32_t* last_ids,
    float* v_render_rgb, float* v_render_depth, const float* v_render_T,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb,
    const float* weight_map, float* o_accum_weight, float* o_accum_weight_den) {
    RawScreen screen((int64_t)I * N, xy, depth, conic, opac, rgb);
    RawScreen v_screen((int64_t)I * N, v_xy, v_depth, v_conic, v_opac, v_rgb);
    RefPrim::WorldBuffer world, v_world;
    RenderOutput::Buffer out, dist, v_out, v_dist;
    out.rgbs = (float3*)render_rgb; out.depths = render_depth;
    v_out.rgbs = (float3*)v_render_rgb; v_out.depths = v_render_depth;
    uint32_t tw = (W + 15) / 16, th = (H + 15) / 16;
#define REF_BWD_ACCUM(MODE) \
    rasterize_to_pixels_bwd_kernel_wrapper<RefPrim, DistortionType::None, MODE, false>( \
        0, I, N, n_isects, nullptr, world, screen, W, H, tw, th, tile_offsets, flatten_ids, \
        render_T, last_ids, out, dist, nullptr, weight_map, v_out, v_render_T, nullptr, v_dist, \
        v_world, v_screen, o_accum_weight, o_accum_weight_den)
    if (mode == 1) REF_BWD_ACCUM(DensifyAccumMode::Max);
    else if (mode == 2) REF_BWD_ACCUM(DensifyAccumMode::Sum);
    else REF_BWD_ACCUM(DensifyAccumMode::Avg);
#undef REF_BWD_ACCUM
    return ref_finish();
}
