// TEST INFRASTRUCTURE.  The reference's tile rasteriser forward kernel, 2D variant
// (src/kernels/raster/RasterizationEval3DFwd_kernel.cuh:48-381 via
// RasterizationFwd_kernel.cuh) for Vanilla3DGS<3>, launched on raw device buffers.
#define NO_TORCH
#include "primitives/Primitive3DGS.cuh"
#include "kernels/raster/RasterizationFwd_kernel.cuh"
#include "ref_common.cuh"
#include "ref_sync.h"

extern "C" int ref_raster_fwd(
    uint32_t I, uint32_t N, uint32_t n_isects, uint32_t W, uint32_t H,
    float* xy, float* depth, float* conic, float* opac, float* rgb,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* out_rgb, float* out_depth, float* out_T, int32_t* last_ids) {
    RawScreen screen((int64_t)I * N, xy, depth, conic, opac, rgb);
    RefPrim::WorldBuffer world;
    RenderOutput::Buffer out, dist;
    out.rgbs = (float3*)out_rgb; out.depths = out_depth;
    uint32_t tw = (W + 15) / 16, th = (H + 15) / 16;
    rasterize_to_pixels_fwd_kernel_wrapper<RefPrim, DistortionType::None, false>(
        0, I, N, n_isects, nullptr, world, screen, W, H, tw, th, tile_offsets, flatten_ids, out, out_T, last_ids, dist, nullptr);
    return ref_finish();
}
