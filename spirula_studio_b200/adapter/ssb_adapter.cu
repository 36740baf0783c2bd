// Adapter between spirula-studio's kernel-launch seam and libssb_b200.
//
// This translation unit is compiled INSIDE the reference tree's include path (-I<reference>/src): it includes the
// reference's own headers and DEFINES the free functions they declare, with the reference's signatures, on top of the
// C ABI of include/ssb.h.  Linked in place of the reference's src/kernels/{projection,tile,raster}/*.cu (and the
// src/instantiations/*.cu they pull in), it lets src/engine compile and link unchanged for the path this library covers:
//
//   projection_3dgs_forward        (src/kernels/projection/ProjectionFwd.cuh:17-34)   -> ssb_project_fwd + ssb_screen_unpack
//   compute_tile_active            (src/kernels/tile/IntersectTile.cuh:18-22)        -> ssb_tile_active
//   do_intersect_tile_generic      (src/kernels/tile/IntersectTile.cuh:24-40)        -> ssb_screen_pack + ssb_intersect_tiles_live
//   rasterize_to_pixels_3dgs_fwd   (src/kernels/raster/RasterizationFwd.cuh:16-37)    -> ssb_screen_pack + ssb_raster_fwd
//   rasterize_to_pixels_3dgs_bwd   (src/kernels/raster/RasterizationBwd.cuh:18-48)    -> ssb_raster_bwd_accum + unpack of the gradient records
//   projection_3dgs_backward       (src/kernels/projection/ProjectionBwd.cuh:18-46)   -> ssb_screen_pack + ssb_project_bwd / ssb_project_bwd_packed
//   fused_projection_bwd_optimizer_3dgs (src/kernels/optim/FusedProjectionBwdOptim.cuh:19-63) -> ssb_project_bwd_optimize[_q16] (quantisation levels 0 and 1)
//   compute_multi_scale_per_pixel_losses (src/kernels/loss/PerPixelLoss.cuh:160-189)  -> ssb_loss_multi_scale (colour terms only)
//   fused_optim_3dgs_geometry      (src/kernels/optim/Optimizer.cuh:120-144)         -> ssb_adam_step_ex without features_dc
//   fused_adam_step                (src/kernels/optim/Optimizer.cuh:147-158)         -> ssb_adam_plain
//   fused_adam_step_quantized      (src/kernels/optim/Optimizer.cuh:169-181)         -> ssb_adam_step_sh_quantized_ex, fp32 values
//   fused_adam_step_quantized_value (src/kernels/optim/Optimizer.cuh:184-205)        -> ssb_adam_step_sh_quantized_ex
//
// The mip and 3dgut siblings declared in the same headers (and defined in the same reference source files, so they go
// when those files are replaced) are defined here too and throw: the link stays complete, the primitives stay refused.
//
// Outputs are views into the reference's process-global DevicePool under the reference's own PoolSlots, sized exactly as
// the reference sizes them (the pair count is read back to the host where the reference reads it back), so callers see
// the same tensors.  The 48-byte records and workspaces this library works on are scratch of the adapter, kept in the
// pool's dynamically named side map.  What the library does not cover is refused the way the reference refuses bad
// arguments (std::runtime_error, src/core/Common.cuh:133-146): AABB-mode
// intersection, distortion-loss channels, median depth, other primitives.
#include "ssb.h"

#include <kernels/optim/FusedProjectionBwdOptim.cuh>
#include <kernels/projection/ProjectionBwd.cuh>
#include <kernels/projection/ProjectionFwd.cuh>
#include <kernels/raster/RasterizationBwd.cuh>
#include <kernels/raster/RasterizationFwd.cuh>
#include <kernels/tile/IntersectTile.cuh>
#include <kernels/loss/PerPixelLoss.cuh>
#include <kernels/optim/Optimizer.cuh>

#include <stdexcept>
#include <string>

namespace {

void ssb_check(int status) {
    if (status == SSB_OK) return;
    if (status == SSB_ERR_OUT_OF_MEMORY) backend::throw_out_of_memory(0);
    throw std::runtime_error(std::string("libssb_b200: ") + ssb_last_error_string());
}

[[noreturn]] void unsupported(const char* what) {
    throw std::runtime_error(std::string("ssb adapter: ") + what + " is outside the path libssb_b200 covers");
}

// Scratch of the adapter: grow-only, owned by the reference's pool like every other transient buffer.
template <class T>
T* scratch(const char* name, int64_t count, VramCategory cat = VramCategory::SplatXImg) {
    DeviceVector<T> v;
    v.resize_dynamic(cat, std::string("ssb_adapter.") + name, count > 0 ? count : 1);
    return v.data_ptr();
}

int camera_model_of(const std::string& s) {
    switch (cmt(s)) {
        case CameraModelType::PINHOLE: return SSB_CAMERA_PINHOLE;
        case CameraModelType::FISHEYE: return SSB_CAMERA_FISHEYE;
        case CameraModelType::EQUISOLID: return SSB_CAMERA_EQUISOLID;
        case CameraModelType::EQUIRECTANGULAR: return SSB_CAMERA_EQUIRECT;
        default: unsupported("this camera model");
    }
}

// The reference's five ScreenBuffer arrays -> records.  `depths` may stand in for the depth array and `rgb` may be null
// (the intersection needs neither colour nor ray depth).
SsbScreenRec* pack_records(const char* name, const float* xy, const float* depth, const float* conic, const float* opac, const float* rgb, int64_t m) {
    SsbScreenRec* rec = scratch<SsbScreenRec>(name, m);
    ssb_check(ssb_screen_pack(xy, depth, conic, opac, rgb ? rgb : conic, m, rec, nullptr));
    return rec;
}

// Packed pairs -> the dense [view][splat] layout: aabb rows (a zero row = "not visible") and gradient records.
__global__ void scatter_pairs_kernel(int64_t nnz, int64_t n, int32_t n_views, const int32_t* camera_ids, const int32_t* gaussian_ids, const float4* aabb, const float* xy,
                                     const float* depth, const float* conic, const float* opac, const float* rgb, float4* dense_aabb, SsbScreenRec* dense_rec) {
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= nnz) return;
    const int32_t cam = camera_ids[v], gid = gaussian_ids[v];
    if ((uint32_t)cam >= (uint32_t)n_views || (uint64_t)gid >= (uint64_t)n) return;      // an id outside the layout is skipped, never followed
    const int64_t slot = (int64_t)cam * n + gid;
    dense_aabb[slot] = aabb[v];
    float4* r = (float4*)(dense_rec + slot);
    r[0] = make_float4(xy[2 * v], xy[2 * v + 1], 0.f, 0.f);
    r[1] = make_float4(conic[3 * v], conic[3 * v + 1], conic[3 * v + 2], opac[v]);
    r[2] = make_float4(rgb[3 * v], rgb[3 * v + 1], rgb[3 * v + 2], depth[v]);
}

struct WorldArgs {
    SsbSplats splats;
    SsbShQuant shq;
    bool quantised;
};

// The six world arrays (+ quantised SH values) of a reference call as the library's argument structs.
WorldArgs world_args(const char* who, const std::vector<DeviceTensorFloatND>& w, const std::optional<TorchTensorView>& sh_value_packed,
                     const std::optional<TorchTensorView>& sh_value_bounds, uint32_t num_sh_buffer, int sh_value_bits, int64_t sh_bounds_stride) {
    if (w.size() != 6) throw std::runtime_error(std::string(who) + ": expected six world arrays");
    if (sh_value_bits == 32 && Vanilla3DGS<0>::WorldBuffer(w).sh_degree() != 3) unsupported("an SH buffer that does not hold 15 coefficients per splat");
    if (sh_value_bits != 32 && num_sh_buffer != 15) unsupported("a quantised SH buffer that does not hold 15 coefficients");
    WorldArgs a{};
    a.quantised = sh_value_bits != 32;
    a.splats = SsbSplats{w[0].data_ptr(), w[1].data_ptr(), w[2].data_ptr(), w[3].data_ptr(), w[4].data_ptr(), a.quantised ? nullptr : w[5].data_ptr()};
    if (a.quantised) {
        if (!sh_value_packed.has_value() || !sh_value_bounds.has_value()) throw std::runtime_error(std::string(who) + ": quantised SH without its buffers");
        a.shq.packed = (void*)std::get<0>(sh_value_packed.value());
        a.shq.bounds = (float*)std::get<0>(sh_value_bounds.value());
        a.shq.bits = sh_value_bits;
        a.shq.bounds_stride = sh_bounds_stride;
    }
    return a;
}

}  // namespace

std::tuple<DeviceTensor2D<float4>, DeviceTensor2D<float>, std::vector<DeviceTensorFloatND>> projection_3dgs_forward(
    const int64_t num_splats, const int max_sh_degree, const std::vector<DeviceTensorFloatND>& in_splats,
    TorchTensorView viewmats, TorchTensorView intrins, const uint32_t image_width, const uint32_t image_height,
    const std::string camera_model, const std::string distortion, const TorchTensorView dist_coeffs, DeviceVector<float> radii,
    const std::optional<TorchTensorView> sh_value_packed, const std::optional<TorchTensorView> sh_value_bounds,
    const uint32_t num_sh_buffer, const int sh_value_bits, const int64_t sh_bounds_stride) {
    if (in_splats.size() != 6) throw std::runtime_error("projection_3dgs_forward: expected six world arrays");
    const int sh_degree = std::min(Vanilla3DGS<0>::WorldBuffer(in_splats).sh_degree(), max_sh_degree);
    if (sh_degree < 0 || sh_degree > 3) unsupported("an SH degree above 3");
    if (Vanilla3DGS<0>::WorldBuffer(in_splats).sh_degree() != 3) unsupported("an SH buffer that does not hold 15 coefficients per splat");
    if (sh_value_bits != 32 && num_sh_buffer != 15) unsupported("a quantised SH buffer that does not hold 15 coefficients");
    const uint32_t C = (uint32_t)std::get<2>(viewmats)[0];
    const int64_t N = num_splats, m = (int64_t)C * N;

    SsbSplats sp = {in_splats[0].data_ptr(), in_splats[1].data_ptr(), in_splats[2].data_ptr(),
                    in_splats[3].data_ptr(), in_splats[4].data_ptr(), sh_value_bits == 32 ? in_splats[5].data_ptr() : nullptr};
    SsbShQuant shq = {};
    if (sh_value_bits != 32) {
        if (!sh_value_packed.has_value() || !sh_value_bounds.has_value()) throw std::runtime_error("projection_3dgs_forward: quantised SH without its buffers");
        shq.packed = (void*)std::get<0>(sh_value_packed.value());
        shq.bounds = (float*)std::get<0>(sh_value_bounds.value());
        shq.bits = sh_value_bits;
        shq.bounds_stride = sh_bounds_stride;      // 0 = one bound per 256 splats, as in the reference
    }
    SsbCameras cams = {(const float*)std::get<0>(viewmats), (const float*)std::get<0>(intrins), (int32_t)C,
                       (int32_t)image_width, (int32_t)image_height, camera_model_of(camera_model), 0,
                       (int32_t)cdt(distortion), sh_degree + 1, (const float*)std::get<0>(dist_coeffs)};      // a pair the reference does not instantiate: SSB_ERR_UNSUPPORTED, thrown

    DeviceTensor2D<float4> aabb;
    aabb.resize(PoolSlot::ProjAabb, C, N);
    DeviceTensor2D<float> sorting_depths;
    sorting_depths.resize(PoolSlot::ProjDepths, C, N);
    std::vector<DeviceTensorFloatND> screen = Vanilla3DGS<3>::ScreenBuffer::empty_pool(m, PoolSlot::ProjScreen);
    SsbScreenRec* rec = scratch<SsbScreenRec>("proj_records", m);
    ssb_check(ssb_project_fwd(&sp, sh_value_bits != 32 ? &shq : nullptr, N, &cams, (float*)aabb.data_ptr(), sorting_depths.data_ptr(),
                              radii.data_ptr(), rec, nullptr));
    ssb_check(ssb_screen_unpack(rec, m, screen[0].data_ptr(), screen[1].data_ptr(), screen[2].data_ptr(), screen[3].data_ptr(),
                                screen[4].data_ptr(), nullptr));
    return std::make_tuple(aabb, sorting_depths, screen);
}

int64_t intersect_tile_count(int width, int height) {
    return (int64_t)((width + SSB_TILE - 1) / SSB_TILE) * ((height + SSB_TILE - 1) / SSB_TILE);
}

void compute_tile_active(TorchTensorView mask, int I, int width, int height, int32_t* tile_active) {
    const auto& ms = std::get<2>(mask);     // [I, H_mask, W_mask] bool, one byte each
    ssb_check(ssb_tile_active((const uint8_t*)std::get<0>(mask), I, (int32_t)ms[1], (int32_t)ms[2], width, height, tile_active, nullptr));
    backend::device_synchronize();
}

std::tuple<DeviceVector<int64_t>, DeviceVector<int32_t>, DeviceTensor3D<int32_t>> do_intersect_tile_generic(
    DeviceTensorFloatND aabb, DeviceTensorFloatND depths, DeviceTensorFloatND* proj_xy, DeviceTensorFloatND* proj_conic,
    DeviceTensorFloatND* proj_opac, const uint32_t I, TorchTensorView intrins, const uint32_t image_width, const uint32_t image_height,
    DeviceVector<int32_t>* image_ids, const int32_t* tile_active) {
    (void)intrins;
    if (!proj_xy || !proj_conic || !proj_opac) unsupported("AABB-mode tile intersection");
    const int64_t total = depths.numel();
    const uint32_t tw = (image_width + SSB_TILE - 1) / SSB_TILE, th = (image_height + SSB_TILE - 1) / SSB_TILE;
    const int64_t n_tiles = (int64_t)tw * th * I;

    DeviceTensor3D<int32_t> offsets;
    offsets.resize(PoolSlot::IsectOffsets, I, th, tw);
    if (total == 0) {
        offsets.zero();
        return std::make_tuple(DeviceVector<int64_t>{}, DeviceVector<int32_t>{}, offsets);
    }
    SsbScreenRec* rec = pack_records("isect_records", proj_xy->data_ptr(), depths.data_ptr(), proj_conic->data_ptr(), proj_opac->data_ptr(), nullptr, total);
    int64_t* d_count = scratch<int64_t>("isect_count", 2);
    // The library keeps the pair count on the device and works inside a caller-chosen capacity; the reference's contract is
    // exact sizes, so the count comes back to the host here (as the reference's own launcher does) and a capacity that
    // turned out too small is grown and the call repeated.
    static int64_t pairs_per_record = 8;
    for (;;) {
        const int64_t cap = std::max<int64_t>(pairs_per_record * total, 1024);
        const int64_t ws_bytes = ssb_intersect_tiles_workspace_bytes(n_tiles, cap);
        void* ws = scratch<unsigned char>("isect_workspace", ws_bytes);
        int64_t* keys = scratch<int64_t>("isect_keys", cap);
        int32_t* flat = scratch<int32_t>("isect_flat", cap);
        if (image_ids) {
            backend::memcpy_sync(d_count + 1, &total, sizeof(int64_t), backend::MemcpyKind::HostToDevice);      // the pair count, which the library reads on the device
            ssb_check(ssb_intersect_tiles_packed_live((const float*)aabb.data_ptr(), depths.data_ptr(), rec, image_ids->data_ptr(), d_count + 1, total, (int32_t)I,
                                                      (int32_t)image_width, (int32_t)image_height, ws, ws_bytes, keys, flat, cap, offsets.data_ptr(), d_count,
                                                      tile_active, nullptr));
        } else
            ssb_check(ssb_intersect_tiles_live((const float*)aabb.data_ptr(), depths.data_ptr(), rec, total, total / I, (int32_t)image_width,
                                               (int32_t)image_height, ws, ws_bytes, keys, flat, cap, offsets.data_ptr(), d_count, tile_active, nullptr));
        int64_t n_isects = 0;
        backend::memcpy_sync(&n_isects, d_count, sizeof(int64_t), backend::MemcpyKind::DeviceToHost);
        int32_t bits = 0;
        ssb_device_status(&bits, nullptr);          // clears the "pairs dropped" flag a too-small first try raised
        if (n_isects > cap) { pairs_per_record = (n_isects + total - 1) / total + 1; continue; }
        if (n_isects == 0) {
            offsets.zero();
            return std::make_tuple(DeviceVector<int64_t>{}, DeviceVector<int32_t>{}, offsets);
        }
        DeviceVector<int64_t> isect_ids;
        isect_ids.resize(PoolSlot::IsectIdsA, n_isects);
        DeviceVector<int32_t> flatten_ids;
        flatten_ids.resize(PoolSlot::IsectFlatA, n_isects);
        backend::memcpy_sync(isect_ids.data_ptr(), keys, n_isects * sizeof(int64_t), backend::MemcpyKind::DeviceToDevice);
        backend::memcpy_sync(flatten_ids.data_ptr(), flat, n_isects * sizeof(int32_t), backend::MemcpyKind::DeviceToDevice);
        return std::make_tuple(isect_ids, flatten_ids, offsets);
    }
}

std::tuple<RenderOutput::TensorTuple, DeviceTensor3D<float>, DeviceTensor3D<int32_t>, RenderOutput::TensorTuple, DeviceTensor3D<float>>
rasterize_to_pixels_3dgs_fwd(int64_t num_splats, std::vector<DeviceTensorFloatND> splats_w, std::vector<DeviceTensorFloatND> splats_s,
                             DeviceVector<int32_t> gaussian_ids, const uint32_t image_width, const uint32_t image_height,
                             const DeviceTensor3D<int32_t> tile_offsets, const DeviceVector<int32_t> flatten_ids, DistortionType dist_type,
                             bool output_median) {
    (void)num_splats; (void)splats_w; (void)gaussian_ids;      // the rasteriser addresses records through the flatten ids alone
    if (dist_type != DistortionType::None) unsupported("a distortion-loss channel");
    if (output_median) unsupported("the median-depth output");
    if (splats_s.size() != 5) throw std::runtime_error("rasterize_to_pixels_3dgs_fwd: expected five screen arrays");
    const int64_t batch = tile_offsets.size<0>();
    const int64_t m = splats_s[1].numel();
    RenderOutput::TensorTuple renders, distortions;
    RenderOutput::resize<Vanilla3DGS<0>::pixelType>(renders, batch, image_height, image_width, PoolSlot::Renders);
    DeviceTensor3D<float> render_Ts;
    DeviceTensor3D<int32_t> render_last_ids;
    render_Ts.resize(PoolSlot::RenderTs, batch, image_height, image_width);
    render_last_ids.resize(PoolSlot::RenderLastIds, batch, image_height, image_width);
    SsbScreenRec* rec = pack_records("raster_records", splats_s[0].data_ptr(), splats_s[1].data_ptr(), splats_s[2].data_ptr(),
                                     splats_s[3].data_ptr(), splats_s[4].data_ptr(), m);
    int64_t* d_count = scratch<int64_t>("raster_count", 2);
    const int64_t n_isects = flatten_ids.size();
    backend::memcpy_sync(d_count, &n_isects, sizeof(int64_t), backend::MemcpyKind::HostToDevice);
    if (n_isects == 0) {      // nothing to blend: the library still writes T = 1 and zero colour, from an empty list
        static int32_t* none = scratch<int32_t>("raster_empty_list", 4);
        ssb_check(ssb_raster_fwd(rec, m, tile_offsets.data_ptr(), none, 0, d_count, (int32_t)batch, (int32_t)image_width, (int32_t)image_height,
                                 (float*)std::get<0>(renders).data_ptr(), std::get<1>(renders).data_ptr(), render_Ts.data_ptr(),
                                 render_last_ids.data_ptr(), nullptr));
    } else {
        ssb_check(ssb_raster_fwd(rec, m, tile_offsets.data_ptr(), flatten_ids.data_ptr(), n_isects, d_count, (int32_t)batch, (int32_t)image_width,
                                 (int32_t)image_height, (float*)std::get<0>(renders).data_ptr(), std::get<1>(renders).data_ptr(),
                                 render_Ts.data_ptr(), render_last_ids.data_ptr(), nullptr));
    }
    return std::make_tuple(renders, render_Ts, render_last_ids, distortions, DeviceTensor3D<float>{});
}

std::tuple<std::vector<DeviceTensorFloatND>, std::vector<DeviceTensorFloatND>, DeviceVector<float>> rasterize_to_pixels_3dgs_bwd(
    int64_t num_splats, std::vector<DeviceTensorFloatND> splats_w, std::vector<DeviceTensorFloatND> splats_s, DeviceVector<int32_t> gaussian_ids,
    const uint32_t image_width, const uint32_t image_height, const DeviceTensor3D<int32_t> tile_offsets, const DeviceVector<int32_t> flatten_ids,
    const DeviceTensor3D<float> render_Ts, const DeviceTensor3D<int32_t> last_ids, RenderOutput::TensorTuple render_outputs_tuple,
    std::optional<RenderOutput::TensorTuple> distortion_fwd_outputs, DistortionType dist_type, DeviceTensor3D<float> accum_weight_map,
    DensifyAccumMode accum_mode, RenderOutput::TensorTuple v_render_outputs, const DeviceTensor3D<float> v_render_Ts,
    const DeviceTensor3D<float> v_median, std::optional<RenderOutput::TensorTuple> v_distortion_outputs,
    std::optional<std::vector<DeviceTensorFloatND>> v_splats_w, std::optional<std::vector<DeviceTensorFloatND>> v_splats_s) {
    (void)distortion_fwd_outputs; (void)v_distortion_outputs;
    if (dist_type != DistortionType::None) unsupported("a distortion-loss channel");
    if (v_median.data_ptr() != nullptr) unsupported("the median-depth cotangent");
    if (splats_s.size() != 5) throw std::runtime_error("rasterize_to_pixels_3dgs_bwd: expected five screen arrays");
    // as the reference: fresh zeroed gradient arrays unless the caller brings its own to accumulate into
    if (!v_splats_w.has_value()) v_splats_w = Vanilla3DGS<0>::WorldBuffer::zeros_pool(splats_w, PoolSlot::RasterBwdVWorld);
    if (!v_splats_s.has_value()) v_splats_s = Vanilla3DGS<0>::ScreenBuffer::zeros_pool(splats_s, PoolSlot::RasterBwdVScreen);
    if (accum_weight_map.data_ptr() == nullptr) accum_mode = DensifyAccumMode::None;      // no map, nothing to accumulate
    const int64_t batch = tile_offsets.size<0>();
    const int64_t m = splats_s[1].numel();
    DeviceVector<float> o_accum_weight;
    if (accum_any(accum_mode)) {
        o_accum_weight.resize(PoolSlot::RasterBwdAccumWeight, num_splats * accum_lanes(accum_mode));
        o_accum_weight.zero();
    }
    float* aw = o_accum_weight.data_ptr();
    float* aw_den = accum_mode == DensifyAccumMode::Avg ? aw + num_splats : nullptr;
    const int mode = accum_mode == DensifyAccumMode::Max ? SSB_ACCUM_MAX : accum_mode == DensifyAccumMode::Sum ? SSB_ACCUM_SUM
                   : accum_mode == DensifyAccumMode::Avg ? SSB_ACCUM_AVG : SSB_ACCUM_NONE;

    SsbScreenRec* rec = pack_records("raster_records", splats_s[0].data_ptr(), splats_s[1].data_ptr(), splats_s[2].data_ptr(),
                                     splats_s[3].data_ptr(), splats_s[4].data_ptr(), m);
    SsbScreenRec* v_rec = scratch<SsbScreenRec>("raster_grad_records", m);
    backend::memset_sync(v_rec, 0, (size_t)m * sizeof(SsbScreenRec));
    int64_t* d_count = scratch<int64_t>("raster_count", 2);
    const int64_t n_isects = flatten_ids.size();
    backend::memcpy_sync(d_count, &n_isects, sizeof(int64_t), backend::MemcpyKind::HostToDevice);
    if (n_isects > 0) {
        ssb_check(ssb_raster_bwd_accum(rec, m, tile_offsets.data_ptr(), flatten_ids.data_ptr(), n_isects, d_count, (int32_t)batch, (int32_t)image_width,
                                       (int32_t)image_height, std::get<1>(render_outputs_tuple).data_ptr(), render_Ts.data_ptr(), last_ids.data_ptr(),
                                       (const float*)std::get<0>(v_render_outputs).data_ptr(), std::get<1>(v_render_outputs).data_ptr(),
                                       v_render_Ts.data_ptr(), v_rec, mode, accum_weight_map.data_ptr(), num_splats,
                                       gaussian_ids.data_ptr(), aw, aw_den, nullptr));
        // gradient records -> the five gradient arrays, added to what they hold (zeros, or the caller's running sums)
        std::vector<DeviceTensorFloatND>& v = v_splats_s.value();
        ssb_check(ssb_screen_unpack_add(v_rec, m, v[0].data_ptr(), v[1].data_ptr(), v[2].data_ptr(), v[3].data_ptr(), v[4].data_ptr(), nullptr));
    }
    return std::make_tuple(v_splats_w.value(), v_splats_s.value(), o_accum_weight);
}


// ---- loss ---------------------------------------------------------------------------------------------------------------

LossValues compute_multi_scale_per_pixel_losses(
    int num_loss_scales, TorchTensorView render_rgb, TorchTensorView ref_rgb, TorchTensorView render_depth, TorchTensorView ref_depth,
    TorchTensorView render_normal, TorchTensorView depth_normal, TorchTensorView ref_normal, TorchTensorView render_Ts, TorchTensorView rgb_dist,
    TorchTensorView depth_dist, TorchTensorView normal_dist, TorchTensorView median_depth, TorchTensorView median_normal, TorchTensorView ref_alpha,
    bool has_mask, const std::array<float, (int)LossWeightIndex::length> loss_weights, const float w_ssim, TorchTensorView v_losses,
    std::vector<bool> needs_input_grad, long num_train_images, TorchTensorView camera_indices, TorchTensorView loss_map_out, int loss_map_mode,
    float robust_edge_aware_quantile, float nms_falloff, PerPixelGrads& grads_out) {
    (void)render_depth; (void)ref_depth; (void)render_normal; (void)depth_normal; (void)ref_normal; (void)render_Ts; (void)rgb_dist; (void)depth_dist;
    (void)normal_dist; (void)median_depth; (void)median_normal; (void)v_losses; (void)num_train_images; (void)robust_edge_aware_quantile; (void)nms_falloff;
    // the library computes the colour terms; every other term must be switched off by its weight
    for (int i = 0; i < (int)LossWeightIndex::length; ++i)
        if (i != (int)LossWeightIndex::RgbSupL1 && loss_weights[i] != 0.0f) unsupported("a loss term other than RGB L1 and SSIM");
    if (std::get<0>(camera_indices)) unsupported("per-camera loss bookkeeping (camera_indices)");
    for (size_t i = 1; i < needs_input_grad.size(); ++i)
        if (needs_input_grad[i]) unsupported("a gradient other than the rendered colour's");
    if (needs_input_grad.empty() || !needs_input_grad[0] || !std::get<0>(grads_out.v_render_rgb)) unsupported("a loss call without the colour gradient");
    const auto& shp = std::get<2>(render_rgb);
    const int32_t B = (int32_t)shp[0], H = (int32_t)shp[1], W = (int32_t)shp[2];
    SsbLossConfig cfg{};
    cfg.w_l1 = loss_weights[(int)LossWeightIndex::RgbSupL1];
    cfg.w_ssim = w_ssim;
    cfg.num_scales = num_loss_scales;
    cfg.loss_map_mode = std::get<0>(loss_map_out) ? loss_map_mode : 0;
    if (has_mask && std::get<0>(ref_alpha)) {
        const auto& ms = std::get<2>(ref_alpha);
        cfg.d_mask = (const uint8_t*)std::get<0>(ref_alpha);          // bool, one byte each
        cfg.mask_h = (int32_t)ms[1];
        cfg.mask_w = (int32_t)ms[2];
    }
    const int64_t ws_bytes = ssb_loss_workspace_bytes(B, H, W, &cfg);
    if (ws_bytes < 0) ssb_check((int)ws_bytes);
    void* ws = scratch<unsigned char>("loss_workspace", ws_bytes, VramCategory::Image);
    float* d_losses = scratch<float>("loss_scalars", 4, VramCategory::Image);
    ssb_check(ssb_loss_multi_scale((const float*)std::get<0>(render_rgb), (const float*)std::get<0>(ref_rgb), B, H, W, &cfg,
                                   (float*)std::get<0>(grads_out.v_render_rgb), d_losses, (float*)std::get<0>(loss_map_out), ws, ws_bytes, nullptr));
    // The reference hands back the scalars of the previous call without waiting (PerPixelLoss.cu:1346-1372); the adapter waits
    // for this call's instead, which a caller that only displays them cannot tell apart from a faster GPU.
    float h[3] = {0.f, 0.f, 0.f};
    backend::memcpy_sync(h, d_losses, sizeof(h), backend::MemcpyKind::DeviceToHost);
    LossValues out{};
    out.rgb_loss = cfg.w_l1 * h[0];
    out.ssim = h[1];
    return out;
}

// ---- optimiser ----------------------------------------------------------------------------------------------------------

void fused_optim_3dgs_geometry(
    int64_t num_splats, DeviceVector<float3> means, DeviceVector<float3> v_means, DeviceVector<float3> g1_means, DeviceVector<float3> g2_means,
    DeviceVector<float4> quats, DeviceVector<float4> v_quats, DeviceVector<float4> g1_quats, DeviceVector<float4> g2_quats, DeviceVector<float3> scales,
    DeviceVector<float3> v_scales, DeviceVector<float3> g1_scales, DeviceVector<float3> g2_scales, DeviceVector<float> opacities,
    DeviceVector<float> v_opacities, DeviceVector<float> g1_opacities, DeviceVector<float> g2_opacities, DeviceVector<float3> features_dc,
    DeviceVector<float3> v_features_dc, DeviceVector<float> radii, DeviceVector<float> densify_score, const float lr_means, const float lr_quats,
    const float lr_scales, const float lr_opacs, const float lr_features_dc, const float max_gauss_ratio, const float scale_regularization_weight,
    const float mcmc_opacity_reg_weight, const float mcmc_scale_reg_weight, const float erank_reg_weight, const float erank_reg_weight_s3,
    const float quat_norm_reg_weight, const float sh_reg_weight, bool use_scale_agnostic_mean, NonShQuantState non_sh, GradQuantBuffers gq, int32_t step,
    DeviceVector<int32_t> per_splat_steps, float grad_scale, bool zero_grad) {
    if (gq.means_packed || gq.sh_packed) unsupported("quantised gradients");
    auto f = [](auto& v) { return (float*)v.data_ptr(); };
    SsbAdamExtras ex{};
    ex.max_gauss_ratio = max_gauss_ratio; ex.scale_regularization_weight = scale_regularization_weight;
    ex.mcmc_opacity_reg_weight = mcmc_opacity_reg_weight; ex.mcmc_scale_reg_weight = mcmc_scale_reg_weight;
    ex.erank_reg_weight = erank_reg_weight; ex.erank_reg_weight_s3 = erank_reg_weight_s3; ex.quat_norm_reg_weight = quat_norm_reg_weight;
    ex.use_scale_agnostic_mean = use_scale_agnostic_mean ? 1 : 0;
    ex.d_radii = radii.data_ptr(); ex.d_steps = per_splat_steps.data_ptr(); ex.n_total = num_splats; ex.d_densify_score = densify_score.data_ptr();
    if (non_sh.enabled) {
        // moments of all five arrays in 16-bit codes; DC is updated in the same launch with sh_reg_weight as its regulariser
        SsbSplats p{f(means), f(quats), f(scales), f(opacities), f(features_dc), nullptr};
        SsbSplats g{f(v_means), f(v_quats), f(v_scales), f(v_opacities), f(v_features_dc), nullptr};
        SsbMomentsQ16 mom{{non_sh.means_packed, non_sh.quats_packed, non_sh.scales_packed, non_sh.opacities_packed, non_sh.features_dc_packed},
                          {(float*)non_sh.means_bounds, (float*)non_sh.quats_bounds, (float*)non_sh.scales_bounds, (float*)non_sh.opacities_bounds,
                           (float*)non_sh.features_dc_bounds}};
        SsbAdamConfig cfg{lr_means, lr_quats, lr_scales, lr_opacs, lr_features_dc, 0.f, sh_reg_weight, grad_scale, step, zero_grad ? 1 : 0};
        ssb_check(ssb_adam_step_q16(&p, &g, &mom, 0, num_splats, &cfg, &ex, nullptr));
        return;
    }
    SsbSplats p{f(means), f(quats), f(scales), f(opacities), nullptr, nullptr};
    SsbSplats g{f(v_means), f(v_quats), f(v_scales), f(v_opacities), nullptr, nullptr};
    SsbSplats m1{f(g1_means), f(g1_quats), f(g1_scales), f(g1_opacities), nullptr, nullptr};
    SsbSplats m2{f(g2_means), f(g2_quats), f(g2_scales), f(g2_opacities), nullptr, nullptr};
    SsbAdamConfig cfg{lr_means, lr_quats, lr_scales, lr_opacs, 0.f, 0.f, sh_reg_weight, grad_scale, step, zero_grad ? 1 : 0};    // `step` is the bias-correction exponent: the engine passes its step + 1
    ssb_check(ssb_adam_step_ex(&p, &g, &m1, &m2, 0, num_splats, &cfg, &ex, nullptr));
}

void fused_adam_step(int64_t num_splats, DeviceTensorFloatND param, DeviceTensorFloatND grad, DeviceTensorFloatND exp_avg, DeviceTensorFloatND exp_avg_sq,
                     float lr, int32_t step, DeviceVector<int32_t> per_splat_steps, float l2_reg, float l2_reg_offset, float grad_scale, bool zero_grad) {
    const int64_t numel = param.numel();
    if (num_splats <= 0 || numel == 0) return;
    ssb_check(ssb_adam_plain(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), numel, (int32_t)(numel / num_splats), lr, step,
                             per_splat_steps.data_ptr(), l2_reg, l2_reg_offset, grad_scale, zero_grad ? 1 : 0, nullptr));
}

static SsbAdamConfig sh_config(float lr, int32_t step, float l2_reg, float grad_scale, bool zero_grad) {
    return SsbAdamConfig{0.f, 0.f, 0.f, 0.f, 0.f, lr, l2_reg, grad_scale, step, zero_grad ? 1 : 0};
}

void fused_adam_step_quantized(int64_t num_splats, DeviceTensorFloatND param, DeviceTensorFloatND grad, uint8_t* packed, float4* quant_bounds, float lr,
                               int32_t step, DeviceVector<int32_t> per_splat_steps, float l2_reg, float l2_reg_offset, int bits, float grad_scale,
                               bool zero_grad) {
    const int64_t numel = param.numel();
    if (num_splats <= 0 || numel == 0) return;
    if (l2_reg != 0.0f && l2_reg_offset != 0.0f) unsupported("an L2 offset in the quantised-state Adam step");
    const SsbAdamConfig cfg = sh_config(lr, step, l2_reg, grad_scale, zero_grad);
    ssb_check(ssb_adam_step_sh_quantized_ex(grad.data_ptr(), packed, (float*)quant_bounds, param.data_ptr(), nullptr, 32, bits, 0, numel, numel, &cfg,
                                            per_splat_steps.data_ptr(), (int32_t)(numel / num_splats), nullptr));
}

void fused_adam_step_quantized_value(int64_t num_splats, int64_t param_numel, DeviceTensorFloatND grad, const uint8_t* grad_q_packed,
                                     const float2* grad_q_bounds, uint8_t* optim_packed, float4* optim_bounds, uint8_t* value_packed, float2* value_bounds,
                                     float lr, int32_t step, DeviceVector<int32_t> per_splat_steps, float l2_reg, float l2_reg_offset, int optim_bits,
                                     int value_bits, float grad_scale, bool zero_grad) {
    if (num_splats <= 0 || param_numel == 0) return;
    if (grad_q_packed || grad_q_bounds) unsupported("quantised gradients");
    if (l2_reg != 0.0f && l2_reg_offset != 0.0f) unsupported("an L2 offset in the quantised Adam step");
    const SsbAdamConfig cfg = sh_config(lr, step, l2_reg, grad_scale, zero_grad);
    ssb_check(ssb_adam_step_sh_quantized_ex(grad.data_ptr(), optim_packed, (float*)optim_bounds, value_packed, (float*)value_bounds, value_bits, optim_bits, 0,
                                            param_numel, param_numel, &cfg, per_splat_steps.data_ptr(), (int32_t)(param_numel / num_splats), nullptr));
}


// ---- projection backward ------------------------------------------------------------------------------------------------

void projection_3dgs_backward(
    const int64_t num_splats, const int max_sh_degree, const std::vector<DeviceTensorFloatND>& splats_world, TorchTensorView viewmats,
    TorchTensorView intrins, const uint32_t image_width, const uint32_t image_height, const std::string camera_model, const std::string distortion,
    const TorchTensorView dist_coeffs, const DeviceVector<int32_t> camera_ids, const DeviceVector<int32_t> gaussian_ids, const DeviceTensor2D<float4> aabb,
    const std::vector<DeviceTensorFloatND>& v_splats_screen, const std::vector<DeviceTensorFloatND>& v_splats_world, DeviceTensor2D<float>* v_viewmats,
    const std::optional<TorchTensorView> sh_value_packed, const std::optional<TorchTensorView> sh_value_bounds, const uint32_t num_sh_buffer,
    const int sh_value_bits, const int64_t sh_bounds_stride) {
    if (v_viewmats != nullptr && v_viewmats->data_ptr() != nullptr) unsupported("the camera-pose gradient");
    if (v_splats_screen.size() != 5 || v_splats_world.size() != 6) throw std::runtime_error("projection_3dgs_backward: expected five screen and six world gradient arrays");
    if (max_sh_degree < 0 || max_sh_degree > 3) unsupported("an SH degree above 3");
    const WorldArgs w = world_args("projection_3dgs_backward", splats_world, sh_value_packed, sh_value_bounds, num_sh_buffer, sh_value_bits, sh_bounds_stride);
    const uint32_t C = (uint32_t)std::get<2>(viewmats)[0];
    const int64_t N = num_splats;
    if (N == 0 || C == 0) return;
    SsbCameras cams = {(const float*)std::get<0>(viewmats), (const float*)std::get<0>(intrins), (int32_t)C, (int32_t)image_width, (int32_t)image_height,
                       camera_model_of(camera_model), 0, (int32_t)cdt(distortion), max_sh_degree + 1, (const float*)std::get<0>(dist_coeffs)};
    // gradients are ADDED to the caller's arrays, as the reference's atomics do
    SsbSplats g = {v_splats_world[0].data_ptr(), v_splats_world[1].data_ptr(), v_splats_world[2].data_ptr(), v_splats_world[3].data_ptr(),
                   v_splats_world[4].data_ptr(), v_splats_world[5].data_ptr()};
    const bool packed = camera_ids.data_ptr() && gaussian_ids.data_ptr();
    const int64_t m = packed ? (int64_t)camera_ids.size() : (int64_t)C * N;
    if (m == 0) return;
    SsbScreenRec* v_rec = pack_records("proj_bwd_grad_records", v_splats_screen[0].data_ptr(), v_splats_screen[1].data_ptr(), v_splats_screen[2].data_ptr(),
                                       v_splats_screen[3].data_ptr(), v_splats_screen[4].data_ptr(), m);
    if (!packed) {
        ssb_check(ssb_project_bwd(&w.splats, w.quantised ? &w.shq : nullptr, N, &cams, (const float*)aabb.data_ptr(), v_rec, &g, 1, nullptr));
        return;
    }
    int64_t* d_pairs = scratch<int64_t>("proj_bwd_pairs", 2);
    backend::memcpy_sync(d_pairs, &m, sizeof(int64_t), backend::MemcpyKind::HostToDevice);
    const int64_t ws_bytes = ssb_project_bwd_packed_workspace_bytes(N, (int32_t)C);
    uint8_t* ws = scratch<uint8_t>("proj_bwd_workspace", ws_bytes);
    ssb_check(ssb_project_bwd_packed(&w.splats, w.quantised ? &w.shq : nullptr, N, &cams, (const float*)aabb.data_ptr(), v_rec, camera_ids.data_ptr(),
                                     gaussian_ids.data_ptr(), d_pairs, m, ws, ws_bytes, &g, 1, nullptr));
}

// Quantisation level 0 (fp32 SH values, fp32 moments of every array) and level 1 (16-bit SH values and 8-bit SH optimiser state
// with one bound per 256 splats: SSB_SH_LAYOUT_SPLAT_BLOCKS; with non_sh.enabled the moments of the other arrays in 16-bit codes).
// v_splats_world is not read: for this primitive the rasteriser's backward leaves it zero (only the 3DGUT rasteriser produces
// world gradients).  With packed pairs the aabb rows and screen gradients are first scattered into the dense [view][splat]
// layout the library's kernel walks.
void fused_projection_bwd_optimizer_3dgs(
    const int64_t num_splats, const int max_sh_degree, std::vector<DeviceTensorFloatND> splats_world, TorchTensorView viewmats, TorchTensorView intrins,
    const uint32_t image_width, const uint32_t image_height, const std::string camera_model, const std::string distortion, const TorchTensorView dist_coeffs,
    const DeviceVector<int32_t> camera_ids, const DeviceVector<int32_t> gaussian_ids, DeviceTensorFloatND aabb,
    const std::vector<DeviceTensorFloatND> v_splats_world, const std::vector<DeviceTensorFloatND> v_splats_screen,
    const std::vector<DeviceTensorFloatND> g1_splats_world, const std::vector<DeviceTensorFloatND> g2_splats_world,
    const std::optional<TorchTensorView> sh_packed, const std::optional<TorchTensorView> sh_quant_bounds, const std::optional<TorchTensorView> sh_value_packed,
    const std::optional<TorchTensorView> sh_value_bounds, NonShQuantState non_sh, DeviceVector<float> radii, DeviceVector<float> densify_score,
    const float lr_means, const float lr_quats, const float lr_scales, const float lr_opacs, const float lr_features_dc, const float lr_features_sh,
    const float max_gauss_ratio, const float scale_regularization_weight, const float mcmc_opacity_reg_weight, const float mcmc_scale_reg_weight,
    const float erank_reg_weight, const float erank_reg_weight_s3, const float quat_norm_reg_weight, const float sh_reg_weight, bool use_scale_agnostic_mean,
    bool color_trust_linear, float eps_tr, std::variant<int32_t, TorchTensorView> step, int quantization_level) {
    (void)v_splats_world; (void)eps_tr;
    if (quantization_level != 0 && quantization_level != 1) unsupported("this quantisation level");
    const bool level1 = quantization_level == 1;
    if (!level1 && non_sh.enabled) unsupported("16-bit moments with fp32 SH in the fused backward + optimiser");
    if (level1 && !(sh_packed.has_value() && sh_quant_bounds.has_value() && sh_value_packed.has_value() && sh_value_bounds.has_value()))
        throw std::runtime_error("fused_projection_bwd_optimizer_3dgs: quantisation level 1 without its SH buffers");
    if (color_trust_linear) unsupported("the linear-colour trust region");
    if (max_sh_degree < 0 || max_sh_degree > 3) unsupported("an SH degree above 3");
    if (v_splats_screen.size() != 5 || g1_splats_world.size() != 6 || g2_splats_world.size() != 6)
        throw std::runtime_error("fused_projection_bwd_optimizer_3dgs: expected five screen gradient arrays and six arrays per moment");
    if (splats_world.size() != 6) throw std::runtime_error("fused_projection_bwd_optimizer_3dgs: expected six world arrays");
    WorldArgs w{};
    if (level1) w.splats = SsbSplats{splats_world[0].data_ptr(), splats_world[1].data_ptr(), splats_world[2].data_ptr(), splats_world[3].data_ptr(),
                                     splats_world[4].data_ptr(), nullptr};
    else w = world_args("fused_projection_bwd_optimizer_3dgs", splats_world, std::nullopt, std::nullopt, 15, 32, 0);
    const uint32_t C = (uint32_t)std::get<2>(viewmats)[0];
    const int64_t N = num_splats, dense = (int64_t)C * N;
    if (N == 0) return;
    SsbCameras cams = {(const float*)std::get<0>(viewmats), (const float*)std::get<0>(intrins), (int32_t)C, (int32_t)image_width, (int32_t)image_height,
                       camera_model_of(camera_model), 0, (int32_t)cdt(distortion), max_sh_degree + 1, (const float*)std::get<0>(dist_coeffs)};
    const float* d_aabb = aabb.data_ptr();
    SsbScreenRec* v_rec = nullptr;
    if (camera_ids.data_ptr() && gaussian_ids.data_ptr()) {
        const int64_t nnz = (int64_t)camera_ids.size();
        float4* dense_aabb = scratch<float4>("fpbo_dense_aabb", dense);
        v_rec = scratch<SsbScreenRec>("fpbo_grad_records", dense);
        backend::memset_sync(dense_aabb, 0, (size_t)dense * sizeof(float4));
        if (nnz > 0) {
            scatter_pairs_kernel<<<(unsigned)((nnz + 255) / 256), 256>>>(nnz, N, (int32_t)C, camera_ids.data_ptr(), gaussian_ids.data_ptr(), (const float4*)aabb.data_ptr(),
                                                                         v_splats_screen[0].data_ptr(), v_splats_screen[1].data_ptr(), v_splats_screen[2].data_ptr(),
                                                                         v_splats_screen[3].data_ptr(), v_splats_screen[4].data_ptr(), dense_aabb, v_rec);
            if (cudaGetLastError() != cudaSuccess) throw std::runtime_error("fused_projection_bwd_optimizer_3dgs: scatter launch failed");
        }
        d_aabb = (const float*)dense_aabb;
    } else {
        v_rec = pack_records("fpbo_grad_records", v_splats_screen[0].data_ptr(), v_splats_screen[1].data_ptr(), v_splats_screen[2].data_ptr(),
                             v_splats_screen[3].data_ptr(), v_splats_screen[4].data_ptr(), dense);
    }
    auto six = [](const std::vector<DeviceTensorFloatND>& v) {
        return SsbSplats{v[0].data_ptr(), v[1].data_ptr(), v[2].data_ptr(), v[3].data_ptr(), v[4].data_ptr(), v[5].data_ptr()};
    };
    SsbSplats m1 = six(g1_splats_world), m2 = six(g2_splats_world);
    SsbAdamExtras ex{};
    ex.max_gauss_ratio = max_gauss_ratio; ex.scale_regularization_weight = scale_regularization_weight;
    ex.mcmc_opacity_reg_weight = mcmc_opacity_reg_weight; ex.mcmc_scale_reg_weight = mcmc_scale_reg_weight;
    ex.erank_reg_weight = erank_reg_weight; ex.erank_reg_weight_s3 = erank_reg_weight_s3; ex.quat_norm_reg_weight = quat_norm_reg_weight;
    ex.use_scale_agnostic_mean = use_scale_agnostic_mean ? 1 : 0;
    ex.d_radii = radii.data_ptr(); ex.n_total = N; ex.d_densify_score = densify_score.data_ptr();
    int32_t scalar_step = 1;
    if (const int32_t* s = std::get_if<int32_t>(&step)) scalar_step = *s;
    else ex.d_steps = (const int32_t*)std::get<0>(std::get<TorchTensorView>(step));
    // this function of the reference takes no gradient scale
    SsbAdamConfig cfg{lr_means, lr_quats, lr_scales, lr_opacs, lr_features_dc, lr_features_sh, sh_reg_weight, 1.0f, scalar_step, 0};
    const int64_t ws_bytes = ssb_project_bwd_optimize_workspace_bytes(N);
    uint8_t* ws = scratch<uint8_t>("fpbo_workspace", ws_bytes + 256);
    ws = (uint8_t*)(((uintptr_t)ws + 255) & ~(uintptr_t)255);
    if (!level1) {
        ssb_check(ssb_project_bwd_optimize(&w.splats, nullptr, N, &cams, d_aabb, v_rec, &m1, &m2, nullptr, &cfg, &ex, ws, ws_bytes, nullptr));
        return;
    }
    SsbSplats p = w.splats;
    p.features_sh = nullptr; m1.features_sh = nullptr; m2.features_sh = nullptr;        // SH lives in the codes
    SsbShQuant shq = {};
    shq.packed = (void*)std::get<0>(sh_value_packed.value()); shq.bounds = (float*)std::get<0>(sh_value_bounds.value());
    shq.bits = 16; shq.bounds_stride = 0;
    SsbShAdamState st = {(uint8_t*)std::get<0>(sh_packed.value()), (float*)std::get<0>(sh_quant_bounds.value()), shq.packed, shq.bounds, 16, 8,
                         SSB_SH_LAYOUT_SPLAT_BLOCKS};
    if (non_sh.enabled) {
        SsbMomentsQ16 mom{{non_sh.means_packed, non_sh.quats_packed, non_sh.scales_packed, non_sh.opacities_packed, non_sh.features_dc_packed},
                          {(float*)non_sh.means_bounds, (float*)non_sh.quats_bounds, (float*)non_sh.scales_bounds, (float*)non_sh.opacities_bounds,
                           (float*)non_sh.features_dc_bounds}};
        ssb_check(ssb_project_bwd_optimize_q16(&p, &shq, N, &cams, d_aabb, v_rec, &mom, nullptr, nullptr, &st, &cfg, &ex, ws, ws_bytes, nullptr));
    } else {
        ssb_check(ssb_project_bwd_optimize(&p, &shq, N, &cams, d_aabb, v_rec, &m1, &m2, &st, &cfg, &ex, ws, ws_bytes, nullptr));
    }
}


// ---- the other primitives of the replaced source files: defined so that the engine links, refused when called ----------------
#define SSB_PROJ_FWD_PARAMS                                                                                                          \
    const int64_t, const int, const std::vector<DeviceTensorFloatND>&, TorchTensorView, TorchTensorView, const uint32_t, const uint32_t, \
        const std::string, const std::string, const TorchTensorView, DeviceVector<float>, const std::optional<TorchTensorView>,          \
        const std::optional<TorchTensorView>, const uint32_t, const int, const int64_t
#define SSB_PROJ_BWD_PARAMS                                                                                                          \
    const int64_t, const int, const std::vector<DeviceTensorFloatND>&, TorchTensorView, TorchTensorView, const uint32_t, const uint32_t, \
        const std::string, const std::string, const TorchTensorView, const DeviceVector<int32_t>, const DeviceVector<int32_t>,           \
        const DeviceTensor2D<float4>, const std::vector<DeviceTensorFloatND>&, const std::vector<DeviceTensorFloatND>&,                  \
        DeviceTensor2D<float>*, const std::optional<TorchTensorView>, const std::optional<TorchTensorView>, const uint32_t, const int,   \
        const int64_t
#define SSB_FPBO_PARAMS                                                                                                              \
    const int64_t, const int, std::vector<DeviceTensorFloatND>, TorchTensorView, TorchTensorView, const uint32_t, const uint32_t,       \
        const std::string, const std::string, const TorchTensorView, const DeviceVector<int32_t>, const DeviceVector<int32_t>,           \
        DeviceTensorFloatND, const std::vector<DeviceTensorFloatND>, const std::vector<DeviceTensorFloatND>,                             \
        const std::vector<DeviceTensorFloatND>, const std::vector<DeviceTensorFloatND>, const std::optional<TorchTensorView>,            \
        const std::optional<TorchTensorView>, const std::optional<TorchTensorView>, const std::optional<TorchTensorView>,               \
        NonShQuantState, DeviceVector<float>, DeviceVector<float>, const float, const float, const float, const float, const float,      \
        const float, const float, const float, const float, const float, const float, const float, const float, const float, bool, bool, \
        float, std::variant<int32_t, TorchTensorView>, int

std::tuple<DeviceTensor2D<float4>, DeviceTensor2D<float>, std::vector<DeviceTensorFloatND>> projection_mip_forward(SSB_PROJ_FWD_PARAMS) { unsupported("the mip primitive"); }
std::tuple<DeviceTensor2D<float4>, DeviceTensor2D<float>, std::vector<DeviceTensorFloatND>> projection_3dgut_forward(SSB_PROJ_FWD_PARAMS) { unsupported("the 3dgut primitive"); }
void projection_mip_backward(SSB_PROJ_BWD_PARAMS) { unsupported("the mip primitive"); }
void projection_3dgut_backward(SSB_PROJ_BWD_PARAMS) { unsupported("the 3dgut primitive"); }
void fused_projection_bwd_optimizer_mip(SSB_FPBO_PARAMS) { unsupported("the mip primitive"); }
void fused_projection_bwd_optimizer_3dgut(SSB_FPBO_PARAMS) { unsupported("the 3dgut primitive"); }
std::tuple<RenderOutput::TensorTuple, DeviceTensor3D<float>, DeviceTensor3D<int32_t>, RenderOutput::TensorTuple, DeviceTensor3D<float>>
rasterize_to_pixels_mip_fwd(int64_t, std::vector<DeviceTensorFloatND>, std::vector<DeviceTensorFloatND>, DeviceVector<int32_t>, const uint32_t, const uint32_t,
                            const DeviceTensor3D<int32_t>, const DeviceVector<int32_t>, DistortionType, bool) { unsupported("the mip primitive"); }

// Each name above must be THE function the reference declares, not an overload beside it: taking the address of an
// overloaded name without a target type does not compile.
static_assert(sizeof(&projection_mip_forward) && sizeof(&projection_3dgut_forward) && sizeof(&projection_mip_backward) && sizeof(&projection_3dgut_backward) &&
              sizeof(&fused_projection_bwd_optimizer_mip) && sizeof(&fused_projection_bwd_optimizer_3dgut) && sizeof(&rasterize_to_pixels_mip_fwd) &&
              sizeof(&projection_3dgs_forward) && sizeof(&projection_3dgs_backward) && sizeof(&fused_projection_bwd_optimizer_3dgs) &&
              sizeof(&rasterize_to_pixels_3dgs_fwd) && sizeof(&rasterize_to_pixels_3dgs_bwd) && sizeof(&do_intersect_tile_generic) && sizeof(&compute_tile_active) &&
              sizeof(&compute_multi_scale_per_pixel_losses) && sizeof(&fused_optim_3dgs_geometry) && sizeof(&fused_adam_step) && sizeof(&fused_adam_step_quantized) &&
              sizeof(&fused_adam_step_quantized_value), "adapter definitions match the reference's declarations");
