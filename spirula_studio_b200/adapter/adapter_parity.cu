// Parity driver for the adapter: calls the reference's kernel-launch functions -- through the reference's own
// declarations and tensor types, exactly as src/engine and the reference's parity tools do
// (src/backend/tests/render_parity.cpp:196-300, raster_bwd_parity.cpp:190-325) -- with ssb_adapter.cu supplying their
// definitions, and holds every output against the reference's own kernels run on the same inputs (the launch shims of the
// reference-side library, loaded at run time).  Stage by stage, each stage fed the reference's upstream outputs; tolerances
// are the reference tools' model |d| <= atol + rtol |ref| with a capped violation fraction.
//
//   adapter_parity <path to libssb_ref.so>        exit code 0 = every check passed
#include <kernels/optim/FusedProjectionBwdOptim.cuh>
#include <kernels/projection/ProjectionBwd.cuh>
#include <kernels/projection/ProjectionFwd.cuh>
#include <kernels/raster/RasterizationBwd.cuh>
#include <kernels/raster/RasterizationFwd.cuh>
#include <kernels/tile/IntersectTile.cuh>
#include <kernels/loss/PerPixelLoss.cuh>
#include <kernels/optim/Optimizer.cuh>

#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

using backend::MemcpyKind;

static constexpr int64_t N = 3000;
static constexpr uint32_t C = 2, W = 200, H = 150;
static constexpr int NUM_SH = 15;

template <typename T>
static T* upload(const std::vector<T>& host) {
    T* d = (T*)backend::device_malloc(host.size() * sizeof(T));
    backend::memcpy_sync(d, host.data(), host.size() * sizeof(T), MemcpyKind::HostToDevice);
    return d;
}
template <typename T>
static T* device_zeros(int64_t n) {
    T* d = (T*)backend::device_malloc((size_t)std::max<int64_t>(n, 1) * sizeof(T));
    backend::memset_sync(d, 0, (size_t)std::max<int64_t>(n, 1) * sizeof(T));
    return d;
}
template <typename T>
static std::vector<T> download(const T* d, int64_t n) {
    std::vector<T> h(n);
    if (n) backend::memcpy_sync(h.data(), d, n * sizeof(T), MemcpyKind::DeviceToHost);
    return h;
}
static TorchTensorView ttv(const void* p, std::vector<int64_t> shape) { return std::make_tuple((uint64_t)p, (uint32_t)4, std::move(shape)); }

static int g_failures = 0;
static void report(const char* what, bool ok, double a = 0, double b = 0) {
    std::printf("%-44s %s  (%g, %g)\n", what, ok ? "ok" : "FAILED", a, b);
    if (!ok) ++g_failures;
}
// fraction of elements with |got - ref| > atol + rtol |ref|
static double frac_bad(const std::vector<float>& got, const std::vector<float>& ref, double atol, double rtol, const std::vector<char>* keep = nullptr, int width = 1) {
    int64_t bad = 0, n = 0;
    for (size_t i = 0; i < ref.size(); ++i) {
        if (keep && !(*keep)[i / width]) continue;
        ++n;
        if (!(std::fabs((double)got[i] - (double)ref[i]) <= atol + rtol * std::fabs((double)ref[i]))) ++bad;
    }
    return n ? (double)bad / (double)n : 0.0;
}
static double max_abs(const std::vector<float>& v) { double m = 0; for (float x : v) m = std::max(m, (double)std::fabs(x)); return m; }

// entry points of the reference-side library (oracle/ref_tool/*.cu)
typedef int (*RefProjectFwd)(uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, float*, const uint8_t*, const float*, int, int64_t,
                             const float*, const float*, float*, float*, float*, float*, float*, float*, float*, float*);
typedef int (*RefIntersect)(uint32_t, uint32_t, uint32_t, uint32_t, const float*, const float*, const float*, const float*, const float*, int64_t*, int64_t*,
                            int64_t, int64_t*, int64_t*, int32_t*, int32_t*, int32_t*, int64_t*, int32_t*);
typedef int (*RefRasterFwd)(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, const int32_t*, const int32_t*, float*,
                            float*, float*, int32_t*);
typedef int (*RefRasterBwd)(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, const int32_t*, const int32_t*, float*,
                            float*, const float*, const int32_t*, float*, float*, const float*, float*, float*, float*, float*, float*);

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: adapter_parity <libssb_ref.so>\n"); return 2; }
    void* ref = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (!ref) { std::fprintf(stderr, "cannot load %s: %s\n", argv[1], dlerror()); return 2; }
    auto ref_project_fwd = (RefProjectFwd)dlsym(ref, "ref_project_fwd");
    auto ref_intersect = (RefIntersect)dlsym(ref, "ref_intersect_tile");
    auto ref_raster_fwd = (RefRasterFwd)dlsym(ref, "ref_raster_fwd");
    auto ref_raster_bwd = (RefRasterBwd)dlsym(ref, "ref_raster_bwd");
    if (!ref_project_fwd || !ref_intersect || !ref_raster_fwd || !ref_raster_bwd) { std::fprintf(stderr, "missing entry point in %s\n", argv[1]); return 2; }

    // ---- inputs: the distributions of the reference's own parity tools (src/backend/tests/projection_parity.cpp:60-80)
    std::mt19937 rng(24680u);
    auto uf = [&](float lo, float hi) { return lo + (hi - lo) * (float)(rng() & 0xffffff) / 16777215.0f; };
    std::vector<float> means(N * 3), quats(N * 4), scales(N * 3), opac(N), dc(N * 3), sh(N * NUM_SH * 3);
    for (int64_t i = 0; i < N; i++) {
        for (int k = 0; k < 3; k++) means[3 * i + k] = uf(-4.f, 4.f);
        means[3 * i + 2] = uf(-2.f, 8.f);
        for (int k = 0; k < 4; k++) quats[4 * i + k] = uf(-1.f, 1.f);
        for (int k = 0; k < 3; k++) scales[3 * i + k] = uf(-5.f, -1.5f);
        opac[i] = uf(-3.f, 5.f);
        for (int k = 0; k < 3; k++) dc[3 * i + k] = uf(-0.5f, 1.5f);
    }
    for (auto& v : sh) v = uf(-0.3f, 0.3f);
    const float cy_ = std::cos(0.2f), sy_ = std::sin(0.2f);
    std::vector<float> vm = {1, 0, 0, 0, 0, 1, 0, 0, 0, 0, 1, 4, 0, 0, 0, 1, cy_, 0, sy_, 0.3f, 0, 1, 0, -0.2f, -sy_, 0, cy_, 5.f, 0, 0, 0, 1};
    std::vector<float> intr = {150, 152, 100, 75, 145, 146, 98, 77};
    float *d_means = upload(means), *d_quats = upload(quats), *d_scales = upload(scales), *d_opac = upload(opac), *d_dc = upload(dc), *d_sh = upload(sh);
    float *d_vm = upload(vm), *d_intr = upload(intr);
    float* d_radii = device_zeros<float>(N);
    std::vector<DeviceTensorFloatND> in_splats = {
        DeviceTensorFloatND(ttv(d_means, {N, 3, 1})), DeviceTensorFloatND(ttv(d_quats, {N, 4, 1})), DeviceTensorFloatND(ttv(d_scales, {N, 3, 1})),
        DeviceTensorFloatND(ttv(d_opac, {N, 1, 1})),  DeviceTensorFloatND(ttv(d_dc, {N, 3, 1})),    DeviceTensorFloatND(ttv(d_sh, {N, NUM_SH * 3, 1}))};
    DeviceVector<float> radii(ttv(d_radii, {N, 1}));
    const int64_t m = (int64_t)C * N, P = (int64_t)C * H * W;

    // ---- 1. projection: the adapter through the reference's signature, the reference's kernel through its shim
    auto pout = projection_3dgs_forward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE",
                                        ttv(nullptr, {(int64_t)C, kCameraDistortionParams}), radii, std::nullopt, std::nullopt, 0, 32, 0);
    backend::device_synchronize();
    auto& a_aabb = std::get<0>(pout);
    auto& a_depths = std::get<1>(pout);
    auto& a_screen = std::get<2>(pout);
    float *r_aabb = device_zeros<float>(m * 4), *r_depths = device_zeros<float>(m), *r_radii = device_zeros<float>(N);
    float *r_xy = device_zeros<float>(m * 2), *r_depth = device_zeros<float>(m), *r_conic = device_zeros<float>(m * 3), *r_opac = device_zeros<float>(m),
          *r_rgb = device_zeros<float>(m * 3);
    if (ref_project_fwd(C, (uint32_t)N, W, H, d_means, d_quats, d_scales, d_opac, d_dc, d_sh, nullptr, nullptr, 32, 256, d_vm, d_intr, r_aabb, r_depths, r_radii,
                        r_xy, r_depth, r_conic, r_opac, r_rgb) != 0) { std::fprintf(stderr, "ref_project_fwd failed\n"); return 2; }
    {
        auto ga = download((const float*)a_aabb.data_ptr(), m * 4), ra = download(r_aabb, m * 4);
        std::vector<char> both(m);
        int64_t n_ref = 0, n_diff = 0;
        for (int64_t i = 0; i < m; ++i) {
            const bool kr = ra[4 * i + 2] > ra[4 * i], kg = ga[4 * i + 2] > ga[4 * i];
            n_ref += kr; n_diff += kr != kg; both[i] = kr && kg;
        }
        report("projection: visible set", n_ref > 500 && (double)n_diff / (double)m <= 2e-3, (double)n_ref, (double)n_diff);
        report("projection: aabb", frac_bad(ga, ra, 5e-3, 5e-4, &both, 4) <= 2e-3);
        report("projection: sorting depth", frac_bad(download(a_depths.data_ptr(), m), download(r_depths, m), 5e-3, 5e-4, &both, 1) <= 2e-3);
        const float* rs[5] = {r_xy, r_depth, r_conic, r_opac, r_rgb};
        const int width[5] = {2, 1, 3, 1, 3};
        const char* names[5] = {"projection: xy", "projection: depth", "projection: conic", "projection: opacity", "projection: rgb"};
        for (int k = 0; k < 5; ++k)
            report(names[k], frac_bad(download(a_screen[k].data_ptr(), m * width[k]), download(rs[k], m * width[k]), 5e-3, 5e-4, &both, width[k]) <= 2e-3);
        report("projection: radii", frac_bad(download(d_radii, N), download(r_radii, N), 1e-4, 1e-3) <= 2e-3);
    }

    // ---- 2. tile intersection on the reference's projected arrays
    std::vector<DeviceTensorFloatND> ref_screen = {DeviceTensorFloatND(ttv(r_xy, {m, 2, 1})), DeviceTensorFloatND(ttv(r_depth, {m, 1, 1})),
                                                   DeviceTensorFloatND(ttv(r_conic, {m, 3, 1})), DeviceTensorFloatND(ttv(r_opac, {m, 1, 1})),
                                                   DeviceTensorFloatND(ttv(r_rgb, {m, 3, 1}))};
    DeviceTensorFloatND aabb_nd(ttv(r_aabb, {m, 4, 1})), depths_nd(ttv(r_depths, {m, 1, 1}));
    auto [isect_ids, flatten_ids, tile_offsets] = do_intersect_tile_generic(aabb_nd, depths_nd, &ref_screen[0], &ref_screen[2], &ref_screen[3], C,
                                                                            ttv(d_intr, {(int64_t)C, 4}), W, H, nullptr, nullptr);
    backend::device_synchronize();
    const uint32_t tw = (W + 15) / 16, th = (H + 15) / 16;
    const int64_t cap = 64 * m;
    int64_t *r_tps = device_zeros<int64_t>(m), *r_cum = device_zeros<int64_t>(m), *r_ids_a = device_zeros<int64_t>(cap), *r_ids_b = device_zeros<int64_t>(cap);
    int32_t *r_fl_a = device_zeros<int32_t>(cap), *r_fl_b = device_zeros<int32_t>(cap), *r_offs = device_zeros<int32_t>((int64_t)C * tw * th);
    int64_t M = 0; int32_t sel = 0;
    if (ref_intersect(C, (uint32_t)N, W, H, r_aabb, r_depths, r_xy, r_conic, r_opac, r_tps, r_cum, cap, r_ids_a, r_ids_b, r_fl_a, r_fl_b, r_offs, &M, &sel) != 0) {
        std::fprintf(stderr, "ref_intersect_tile failed\n"); return 2;
    }
    const int64_t* r_ids = sel ? r_ids_b : r_ids_a;
    const int32_t* r_fl = sel ? r_fl_b : r_fl_a;
    {
        report("intersection: pair count", flatten_ids.size() == M, (double)flatten_ids.size(), (double)M);
        bool same = flatten_ids.size() == M;
        if (same) {
            same = download(isect_ids.data_ptr(), M) == download(r_ids, M);
            report("intersection: sorted keys", same);
            report("intersection: flatten ids", download(flatten_ids.data_ptr(), M) == download(r_fl, M));
            report("intersection: tile offsets", download(tile_offsets.data_ptr(), (int64_t)C * tw * th) == download(r_offs, (int64_t)C * tw * th));
        }
    }

    // ---- 3. rasteriser forward on the reference's arrays and lists
    DeviceVector<int32_t> ref_flat(ttv(r_fl, {M, 1}));
    DeviceTensor3D<int32_t> ref_offsets(ttv(r_offs, {(int64_t)C, (int64_t)th, (int64_t)tw, 1}));
    auto rout = rasterize_to_pixels_3dgs_fwd(N, in_splats, ref_screen, DeviceVector<int32_t>{}, W, H, ref_offsets, ref_flat, DistortionType::None, false);
    backend::device_synchronize();
    auto& renders = std::get<0>(rout);
    auto& render_Ts = std::get<1>(rout);
    auto& last_ids = std::get<2>(rout);
    float *rr_rgb = device_zeros<float>(P * 3), *rr_depth = device_zeros<float>(P), *rr_T = device_zeros<float>(P);
    int32_t* rr_last = device_zeros<int32_t>(P);
    if (ref_raster_fwd(C, (uint32_t)N, (uint32_t)M, W, H, r_xy, r_depth, r_conic, r_opac, r_rgb, r_offs, r_fl, rr_rgb, rr_depth, rr_T, rr_last) != 0) {
        std::fprintf(stderr, "ref_raster_fwd failed\n"); return 2;
    }
    {
        auto g = download((const float*)std::get<0>(renders).data_ptr(), P * 3), r = download(rr_rgb, P * 3);
        double worst = 0; int64_t over = 0;
        for (int64_t i = 0; i < P; ++i) {
            double d = 0;
            for (int k = 0; k < 3; ++k) d = std::max(d, (double)std::fabs(g[3 * i + k] - r[3 * i + k]));
            worst = std::max(worst, d); over += d > 1e-4;
        }
        report("raster forward: image", worst <= 5e-3 && (double)over / (double)P <= 2e-3, worst, (double)over);
        report("raster forward: transmittance", frac_bad(download(render_Ts.data_ptr(), P), download(rr_T, P), 5e-3, 0.0) == 0.0);
        report("raster forward: depth", frac_bad(download(std::get<1>(renders).data_ptr(), P), download(rr_depth, P), 5e-3, 1e-3) <= 2e-3);
        auto gl = download(last_ids.data_ptr(), P), rl = download(rr_last, P);
        int64_t nd = 0;
        for (int64_t i = 0; i < P; ++i) nd += gl[i] != rl[i];
        report("raster forward: last ids", (double)nd / (double)P <= 2e-3, (double)nd);
    }

    // ---- 4. rasteriser backward on the reference's forward outputs
    std::vector<float> h_vrgb(P * 3), h_vdepth(P), h_vT(P);
    for (auto& v : h_vrgb) v = uf(-1.f, 1.f);
    for (auto& v : h_vdepth) v = uf(-0.1f, 0.1f);
    for (auto& v : h_vT) v = uf(-0.1f, 0.1f);
    float *d_vrgb = upload(h_vrgb), *d_vdepth = upload(h_vdepth), *d_vT = upload(h_vT);
    auto t3f3 = [&](float* p) { return DeviceTensor3D<float3>(ttv(p, {(int64_t)C, H, W, 3})); };
    auto t3f1 = [&](float* p) { return DeviceTensor3D<float>(ttv(p, {(int64_t)C, H, W, 1})); };
    RenderOutput::TensorTuple ref_renders{t3f3(rr_rgb), t3f1(rr_depth), DeviceTensor3D<float3>{}};
    RenderOutput::TensorTuple v_renders{t3f3(d_vrgb), t3f1(d_vdepth), DeviceTensor3D<float3>{}};
    DeviceTensor3D<int32_t> ref_last(ttv(rr_last, {(int64_t)C, H, W, 1}));
    auto [v_w, v_s, aw_out] = rasterize_to_pixels_3dgs_bwd(N, in_splats, ref_screen, DeviceVector<int32_t>{}, W, H, ref_offsets, ref_flat, t3f1(rr_T), ref_last,
                                                           ref_renders, std::nullopt, DistortionType::None, DeviceTensor3D<float>{}, DensifyAccumMode::None,
                                                           v_renders, t3f1(d_vT), DeviceTensor3D<float>{}, std::nullopt, std::nullopt, std::nullopt);
    backend::device_synchronize();
    float *g_xy = device_zeros<float>(m * 2), *g_depth = device_zeros<float>(m), *g_conic = device_zeros<float>(m * 3), *g_opac = device_zeros<float>(m),
          *g_rgb = device_zeros<float>(m * 3);
    if (ref_raster_bwd(C, (uint32_t)N, (uint32_t)M, W, H, r_xy, r_depth, r_conic, r_opac, r_rgb, r_offs, r_fl, rr_rgb, rr_depth, rr_T, rr_last, d_vrgb, d_vdepth, d_vT,
                       g_xy, g_depth, g_conic, g_opac, g_rgb) != 0) { std::fprintf(stderr, "ref_raster_bwd failed\n"); return 2; }
    {
        const float* rg[5] = {g_xy, g_depth, g_conic, g_opac, g_rgb};
        const int width[5] = {2, 1, 3, 1, 3};
        const char* names[5] = {"raster backward: v_xy", "raster backward: v_depth", "raster backward: v_conic", "raster backward: v_opacity", "raster backward: v_rgb"};
        for (int k = 0; k < 5; ++k) {
            auto r = download(rg[k], m * width[k]);
            report(names[k], frac_bad(download(v_s[k].data_ptr(), m * width[k]), r, 1e-4 * max_abs(r), 2e-3) <= 5e-3, max_abs(r));
        }
    }
    // ---- 4b. projection backward on the reference's aabb and screen gradients: dense and packed pairs
    {
        typedef int (*RefProjectBwd)(uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, float*, const uint8_t*, const float*, int, int64_t,
                                     const float*, const float*, const float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*);
        typedef int (*RefFpbo)(uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, float*, const float*, const float*, const float*,
                               float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*, float*,
                               float*, float*, float*, float*, float*, float*, const float*, const float*, const float*, float, int, int, const int32_t*);
        auto ref_project_bwd = (RefProjectBwd)dlsym(ref, "ref_project_bwd");
        auto ref_fpbo = (RefFpbo)dlsym(ref, "ref_fpbo");
        if (!ref_project_bwd || !ref_fpbo) { std::fprintf(stderr, "missing ref_project_bwd / ref_fpbo\n"); return 2; }
        const int64_t wd[6] = {3, 4, 3, 1, 3, NUM_SH * 3};
        const float* params_h[6] = {means.data(), quats.data(), scales.data(), opac.data(), dc.data(), sh.data()};
        auto six_zeros = [&]() { std::vector<float*> v(6); for (int k = 0; k < 6; ++k) v[k] = device_zeros<float>(N * wd[k]); return v; };
        auto six_nd = [&](const std::vector<float*>& v) {
            std::vector<DeviceTensorFloatND> o;
            for (int k = 0; k < 6; ++k) o.push_back(DeviceTensorFloatND(ttv(v[k], {N, wd[k], 1})));
            return o;
        };
        // Quaternions enter the fused optimiser normalised, as every optimiser step leaves them: in its scale-agnostic mean update the
        // reference's fused kernel hands the stored quaternion to normalized_quat_to_rotmat as it is
        // (src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:525-531) where its unfused kernel, which the library follows, normalises
        // first (src/kernels/optim/FusedGeometryOptim.cu:171,302-306); the two agree on unit quaternions only.
        std::vector<float> unit_quats = quats;
        for (int64_t i = 0; i < N; ++i) {
            float* q = &unit_quats[4 * i];
            const float inv = 1.0f / std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
            for (int k = 0; k < 4; ++k) q[k] *= inv;
        }
        params_h[1] = unit_quats.data();
        auto six_params = [&]() { std::vector<float*> v(6); for (int k = 0; k < 6; ++k) v[k] = upload(std::vector<float>(params_h[k], params_h[k] + N * wd[k])); return v; };
        std::vector<DeviceTensorFloatND> v_screen_nd = {DeviceTensorFloatND(ttv(g_xy, {m, 2, 1})), DeviceTensorFloatND(ttv(g_depth, {m, 1, 1})),
                                                        DeviceTensorFloatND(ttv(g_conic, {m, 3, 1})), DeviceTensorFloatND(ttv(g_opac, {m, 1, 1})),
                                                        DeviceTensorFloatND(ttv(g_rgb, {m, 3, 1}))};
        const auto no_dist = ttv(nullptr, {(int64_t)C, kCameraDistortionParams});
        auto gw_ref = six_zeros();
        if (ref_project_bwd(C, (uint32_t)N, W, H, d_means, d_quats, d_scales, d_opac, d_dc, d_sh, nullptr, nullptr, 32, 256, d_vm, d_intr, r_aabb, g_xy, g_depth, g_conic,
                            g_opac, g_rgb, gw_ref[0], gw_ref[1], gw_ref[2], gw_ref[3], gw_ref[4], gw_ref[5]) != 0) return 2;
        auto gw_a = six_zeros();
        projection_3dgs_backward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE", no_dist, DeviceVector<int32_t>{},
                                 DeviceVector<int32_t>{}, DeviceTensor2D<float4>(ttv(r_aabb, {(int64_t)C, N, 4})), v_screen_nd, six_nd(gw_a), nullptr, std::nullopt,
                                 std::nullopt, 15, 32, 256);
        backend::device_synchronize();
        const char* gnames[6] = {"means", "quats", "scales", "opacities", "features_dc", "features_sh"};
        bool ok = true;
        for (int k = 0; k < 6; ++k) {
            auto r = download(gw_ref[k], N * wd[k]);
            ok = ok && max_abs(r) > 0 && frac_bad(download(gw_a[k], N * wd[k]), r, 1e-4 * max_abs(r), 2e-3) <= 5e-3;
        }
        report("projection_3dgs_backward", ok);
        // the same pairs packed: camera-major, splat-minor, as the packed projection leaves them
        auto h_aabb = download(r_aabb, m * 4);
        std::vector<int32_t> cam_ids, g_ids;
        for (int64_t i = 0; i < m; ++i)
            if (h_aabb[4 * i + 2] > h_aabb[4 * i] && h_aabb[4 * i + 3] > h_aabb[4 * i + 1]) { cam_ids.push_back((int32_t)(i / N)); g_ids.push_back((int32_t)(i % N)); }
        const int64_t nnz = (int64_t)cam_ids.size();
        auto gather = [&](const float* d, int width) {
            auto h = download(d, m * width);
            std::vector<float> o((size_t)nnz * width);
            for (int64_t v = 0; v < nnz; ++v)
                for (int c = 0; c < width; ++c) o[v * width + c] = h[((int64_t)cam_ids[v] * N + g_ids[v]) * width + c];
            return upload(o);
        };
        float *p_aabb = gather(r_aabb, 4), *p_xy = gather(g_xy, 2), *p_depth = gather(g_depth, 1), *p_conic = gather(g_conic, 3), *p_opac = gather(g_opac, 1),
              *p_rgb = gather(g_rgb, 3);
        int32_t *d_cam_ids = upload(cam_ids), *d_g_ids = upload(g_ids);
        std::vector<DeviceTensorFloatND> p_screen_nd = {DeviceTensorFloatND(ttv(p_xy, {nnz, 2, 1})), DeviceTensorFloatND(ttv(p_depth, {nnz, 1, 1})),
                                                        DeviceTensorFloatND(ttv(p_conic, {nnz, 3, 1})), DeviceTensorFloatND(ttv(p_opac, {nnz, 1, 1})),
                                                        DeviceTensorFloatND(ttv(p_rgb, {nnz, 3, 1}))};
        DeviceVector<int32_t> cam_dv(ttv(d_cam_ids, {nnz, 1})), gid_dv(ttv(d_g_ids, {nnz, 1}));
        auto gw_p = six_zeros();
        projection_3dgs_backward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE", no_dist, cam_dv, gid_dv,
                                 DeviceTensor2D<float4>(ttv(p_aabb, {nnz, (int64_t)1, 4})), p_screen_nd, six_nd(gw_p), nullptr, std::nullopt, std::nullopt, 15, 32, 256);
        backend::device_synchronize();
        ok = nnz > 500 && nnz < m;
        for (int k = 0; k < 6; ++k) {
            auto r = download(gw_ref[k], N * wd[k]);
            ok = ok && frac_bad(download(gw_p[k], N * wd[k]), r, 1e-4 * max_abs(r), 2e-3) <= 5e-3;
        }
        report("projection_3dgs_backward, packed pairs", ok, (double)nnz);

        // ---- 4c. projection backward fused with the optimiser against the reference's fused kernel: every option on, step 3, from small moments
        auto noisy6 = [&](float scale, float shift) {
            std::vector<std::vector<float>> v(6);
            for (int k = 0; k < 6; ++k) { v[k].resize(N * wd[k]); for (auto& x : v[k]) x = shift + scale * (uf(0.f, 1.f) - 0.5f); }
            return v;
        };
        auto up6 = [&](const std::vector<std::vector<float>>& h) { std::vector<float*> v(6); for (int k = 0; k < 6; ++k) v[k] = upload(h[k]); return v; };
        const auto h_g1 = noisy6(1e-5f, 0.f), h_g2 = noisy6(1e-10f, 1e-10f);
        std::vector<float> h_radii(N);
        for (auto& x : h_radii) x = uf(0.5f, 40.f);
        std::vector<int32_t> h_steps(N);
        for (auto& x : h_steps) x = 1 + (int32_t)(rng() % 40);
        float* d_rad = upload(h_radii);
        int32_t* d_steps = upload(h_steps);
        const float lrs[6] = {1e-3f, 2e-3f, 5e-3f, 5e-2f, 2.5e-3f, 1.25e-4f};
        const float reg[7] = {3.0f, 0.7f, 0.9f, 1.1f, 0.5f, 0.3f, 0.2f};
        const float sh_reg = 0.05f;
        auto pr = six_params(), zr = six_zeros(), g1r = up6(h_g1), g2r = up6(h_g2);
        if (ref_fpbo(C, (uint32_t)N, W, H, pr[0], pr[1], pr[2], pr[3], pr[4], pr[5], d_vm, d_intr, r_aabb, g_xy, g_depth, g_conic, g_opac, g_rgb, zr[0], zr[1], zr[2],
                     zr[3], zr[4], zr[5], g1r[0], g1r[1], g1r[2], g1r[3], g1r[4], g1r[5], g2r[0], g2r[1], g2r[2], g2r[3], g2r[4], g2r[5], d_rad, lrs, reg, sh_reg, 1, 0,
                     d_steps) != 0) { std::fprintf(stderr, "ref_fpbo failed\n"); return 2; }
        for (int variant = 0; variant < 2; ++variant) {
            auto pa = six_params(), za = six_zeros(), g1a = up6(h_g1), g2a = up6(h_g2);
            const bool pk = variant == 1;
            fused_projection_bwd_optimizer_3dgs(
                N, 3, six_nd(pa), ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE", no_dist, pk ? cam_dv : DeviceVector<int32_t>{},
                pk ? gid_dv : DeviceVector<int32_t>{}, pk ? DeviceTensorFloatND(ttv(p_aabb, {nnz, 4, 1})) : DeviceTensorFloatND(ttv(r_aabb, {m, 4, 1})), six_nd(za),
                pk ? p_screen_nd : v_screen_nd, six_nd(g1a), six_nd(g2a), std::nullopt, std::nullopt, std::nullopt, std::nullopt, NonShQuantState{},
                DeviceVector<float>(ttv(d_rad, {N, 1})), DeviceVector<float>{}, lrs[0], lrs[1], lrs[2], lrs[3], lrs[4], lrs[5], reg[0], reg[1], reg[2], reg[3], reg[4],
                reg[5], reg[6], sh_reg, true, false, 0.f, std::variant<int32_t, TorchTensorView>(ttv(d_steps, {N, 1})), 0);
            backend::device_synchronize();
            ok = true;
            for (int k = 0; k < 6; ++k) {
                auto rp = download(pr[k], N * wd[k]), r1 = download(g1r[k], N * wd[k]), r2 = download(g2r[k], N * wd[k]);
                const double fp = frac_bad(download(pa[k], N * wd[k]), rp, 5e-6, 1e-4), f1 = frac_bad(download(g1a[k], N * wd[k]), r1, 1e-4 * max_abs(r1), 2e-3),
                             f2 = frac_bad(download(g2a[k], N * wd[k]), r2, 1e-4 * max_abs(r2), 4e-3);
                if (!(fp <= 2e-3 && f1 <= 5e-3 && f2 <= 5e-3)) { ok = false; std::printf("  %s: %g %g %g\n", gnames[k], fp, f1, f2); }
            }
            report(pk ? "fused_projection_bwd_optimizer_3dgs, packed" : "fused_projection_bwd_optimizer_3dgs", ok);
        }
        // ---- 4d. the stock configuration: level 1 (16-bit SH values, 8-bit SH state, bounds per 256 splats) with 16-bit moments
        {
            typedef int (*RefFpboL1)(uint32_t, uint32_t, uint32_t, uint32_t, int, float* const*, const float*, const float*, const float*, float* const*,
                                     float* const*, float* const*, float* const*, uint8_t*, float*, uint8_t*, float*, uint8_t* const*, float* const*, const float*,
                                     const float*, const float*, float, int, int, const int32_t*);
            auto ref_fpbo_l1 = (RefFpboL1)dlsym(ref, "ref_fpbo_l1");
            if (!ref_fpbo_l1) { std::fprintf(stderr, "missing ref_fpbo_l1\n"); return 2; }
            const int64_t nb = (N + 255) / 256, cells = N * 45;
            // SH codes with one bound per 256 splats; state and moments start from zero (the codecs' zero state)
            std::vector<uint16_t> codes(cells);
            std::vector<float> vbound(nb * 2);
            for (int64_t b = 0; b < nb; ++b) {
                const int64_t c0 = b * 256 * 45, c1 = std::min(cells, c0 + 256 * 45);
                float lo = 1e30f, hi = -1e30f;
                for (int64_t i = c0; i < c1; ++i) { lo = std::min(lo, sh[i]); hi = std::max(hi, sh[i]); }
                vbound[2 * b] = lo; vbound[2 * b + 1] = hi;
                for (int64_t i = c0; i < c1; ++i) codes[i] = (uint16_t)std::lround(65535.0 * (sh[i] - lo) / std::max(hi - lo, 1e-30f));
            }
            struct Side { std::vector<float*> p, z; uint16_t* vc; float* vb; uint8_t* oc; float* ob; uint8_t* nq[5]; float* nqb[5]; };
            auto make_side = [&]() {
                Side s; s.p = six_params(); s.z = six_zeros(); s.vc = upload(codes); s.vb = upload(vbound);
                s.oc = device_zeros<uint8_t>(cells * 2); s.ob = device_zeros<float>(nb * 4);
                for (int k = 0; k < 5; ++k) { s.nq[k] = device_zeros<uint8_t>(N * wd[k] * 4); s.nqb[k] = device_zeros<float>(nb * 4); }
                return s;
            };
            Side r = make_side(), a = make_side();
            float* unused5[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
            float* vs5[5] = {g_xy, g_depth, g_conic, g_opac, g_rgb};
            if (ref_fpbo_l1(C, (uint32_t)N, W, H, 3, r.p.data(), d_vm, d_intr, r_aabb, vs5, r.z.data(), unused5, unused5, r.oc, r.ob, (uint8_t*)r.vc, r.vb, r.nq, r.nqb,
                            d_rad, lrs, reg, sh_reg, 1, 0, d_steps) != 0) { std::fprintf(stderr, "ref_fpbo_l1 failed\n"); return 2; }
            NonShQuantState nq;
            nq.enabled = true;
            nq.means_packed = a.nq[0]; nq.quats_packed = a.nq[1]; nq.scales_packed = a.nq[2]; nq.opacities_packed = a.nq[3]; nq.features_dc_packed = a.nq[4];
            nq.means_bounds = (float4*)a.nqb[0]; nq.quats_bounds = (float4*)a.nqb[1]; nq.scales_bounds = (float4*)a.nqb[2]; nq.opacities_bounds = (float4*)a.nqb[3];
            nq.features_dc_bounds = (float4*)a.nqb[4];
            auto g1a = six_zeros(), g2a = six_zeros();
            fused_projection_bwd_optimizer_3dgs(
                N, 3, six_nd(a.p), ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE", no_dist, DeviceVector<int32_t>{},
                DeviceVector<int32_t>{}, DeviceTensorFloatND(ttv(r_aabb, {m, 4, 1})), six_nd(a.z), v_screen_nd, six_nd(g1a), six_nd(g2a),
                std::make_tuple((uint64_t)a.oc, (uint32_t)1, std::vector<int64_t>{cells * 2}), ttv(a.ob, {nb, 4}),
                std::make_tuple((uint64_t)a.vc, (uint32_t)1, std::vector<int64_t>{cells * 2}), ttv(a.vb, {nb, 2}), nq, DeviceVector<float>(ttv(d_rad, {N, 1})),
                DeviceVector<float>{}, lrs[0], lrs[1], lrs[2], lrs[3], lrs[4], lrs[5], reg[0], reg[1], reg[2], reg[3], reg[4], reg[5], reg[6], sh_reg, true, false, 0.f,
                std::variant<int32_t, TorchTensorView>(ttv(d_steps, {N, 1})), 1);
            backend::device_synchronize();
            ok = true;
            for (int k = 0; k < 5; ++k) {
                const double fp = frac_bad(download(a.p[k], N * wd[k]), download(r.p[k], N * wd[k]), 5e-6, 1e-4);
                if (!(fp <= 2e-3)) { ok = false; std::printf("  level 1 %s: %g\n", gnames[k], fp); }
            }
            // SH values and the bounds of both SH buffers: as the numbers the codes stand for
            auto va = download(a.vc, cells), vr = download(r.vc, cells);
            auto ba = download(a.vb, nb * 2), br = download(r.vb, nb * 2);
            int64_t far = 0;
            for (int64_t i = 0; i < cells; ++i) {
                const int64_t b = i / (256 * 45);
                const double xa = ba[2 * b] + (ba[2 * b + 1] - ba[2 * b]) * (va[i] / 65535.0), xr = br[2 * b] + (br[2 * b + 1] - br[2 * b]) * (vr[i] / 65535.0);
                far += std::fabs(xa - xr) > 3.0 * (br[2 * b + 1] - br[2 * b]) / 65535.0 + 1e-12;
            }
            const double fb = frac_bad(ba, br, 2e-5, 2e-3) + frac_bad(download(a.ob, nb * 4), download(r.ob, nb * 4), 2e-3, 2e-3);
            report("fused_projection_bwd_optimizer_3dgs, level 1 + 16-bit moments", ok && far * 200 <= cells && fb == 0.0, (double)far, fb);
        }
        bool refused = false;
        try {
            auto pa = six_params(), za = six_zeros(), g1a = up6(h_g1), g2a = up6(h_g2);
            fused_projection_bwd_optimizer_3dgs(N, 3, six_nd(pa), ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE", no_dist,
                                                DeviceVector<int32_t>{}, DeviceVector<int32_t>{}, DeviceTensorFloatND(ttv(r_aabb, {m, 4, 1})), six_nd(za), v_screen_nd,
                                                six_nd(g1a), six_nd(g2a), std::nullopt, std::nullopt, std::nullopt, std::nullopt, NonShQuantState{},
                                                DeviceVector<float>{}, DeviceVector<float>{}, lrs[0], lrs[1], lrs[2], lrs[3], lrs[4], lrs[5], reg[0], 0.f, 0.f, 0.f, 0.f, 0.f,
                                                0.f, 0.f, false, false, 0.f, std::variant<int32_t, TorchTensorView>((int32_t)1), 1);
        } catch (const std::runtime_error&) { refused = true; }
        report("fused backward + optimiser, level 1 without its buffers: refused", refused);
    }
    // ---- 5. what the library does not cover is refused the way the reference refuses bad arguments
    bool threw = false;
    try {     // a pair outside the reference's instantiation table: the reference throws here too
        projection_3dgs_forward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "FISHEYE", "RATIONAL",
                                ttv(nullptr, {(int64_t)C, kCameraDistortionParams}), radii, std::nullopt, std::nullopt, 0, 32, 0);
    } catch (const std::runtime_error&) { threw = true; }
    report("unsupported distortion tier throws", threw);
    // ---- 5a. the SH degree warm-up: max_sh_degree = 1 against the reference's Vanilla3DGS<1> kernel
    {
        typedef int (*RefFwdDeg)(int, uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, float*, const float*, const float*,
                                 float*, float*, float*, float*, float*, float*, float*, float*);
        auto ref_fwd_deg = (RefFwdDeg)dlsym(ref, "ref_project_fwd_deg");
        if (!ref_fwd_deg) { std::fprintf(stderr, "missing ref_project_fwd_deg\n"); return 2; }
        float* d_radii1 = device_zeros<float>(N);
        DeviceVector<float> radii1(ttv(d_radii1, {N, 1}));
        auto dout = projection_3dgs_forward(N, 1, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "NONE",
                                            ttv(nullptr, {(int64_t)C, kCameraDistortionParams}), radii1, std::nullopt, std::nullopt, 0, 32, 0);
        backend::device_synchronize();
        float *q_aabb = device_zeros<float>(m * 4), *q_depths = device_zeros<float>(m), *q_radii = device_zeros<float>(N);
        float *q_xy = device_zeros<float>(m * 2), *q_depth = device_zeros<float>(m), *q_conic = device_zeros<float>(m * 3), *q_opac = device_zeros<float>(m),
              *q_rgb = device_zeros<float>(m * 3);
        if (ref_fwd_deg(1, C, (uint32_t)N, W, H, d_means, d_quats, d_scales, d_opac, d_dc, d_sh, d_vm, d_intr, q_aabb, q_depths, q_radii, q_xy, q_depth, q_conic,
                        q_opac, q_rgb) != 0) { std::fprintf(stderr, "ref_project_fwd_deg failed\n"); return 2; }
        auto ga = download((const float*)std::get<0>(dout).data_ptr(), m * 4), ra = download(q_aabb, m * 4);
        std::vector<char> both(m);
        for (int64_t i = 0; i < m; ++i) both[i] = (ra[4 * i + 2] > ra[4 * i]) && (ga[4 * i + 2] > ga[4 * i]);
        auto rgb1 = download(std::get<2>(dout)[4].data_ptr(), m * 3), rgb3 = download(r_rgb, m * 3), rgbr = download(q_rgb, m * 3);
        double moved = 0.0;
        for (int64_t i = 0; i < m * 3; ++i) if (both[i / 3]) moved = std::max(moved, (double)std::fabs(rgbr[i] - rgb3[i]));
        report("projection with SH degree 1: rgb", moved > 0.01 && frac_bad(rgb1, rgbr, 5e-3, 5e-4, &both, 3) <= 2e-3, moved);
    }
    // ---- 5b. a lens-distortion tier through the reference's signature against the reference's kernel of that variant
    {
        typedef int (*RefFwdDist)(int, int, uint32_t, uint32_t, uint32_t, uint32_t, float*, float*, float*, float*, float*, float*, const float*, const float*,
                                  float*, float*, float*, float*, float*, float*, float*, float*, float*);
        auto ref_fwd_dist = (RefFwdDist)dlsym(ref, "ref_project_fwd_dist");
        if (!ref_fwd_dist) { std::fprintf(stderr, "missing ref_project_fwd_dist\n"); return 2; }
        std::vector<float> rows = {-0.9f, 0.2f, 0.004f, -0.003f, 0.f, 0.f, 0.f, 0.f, 0.3f, -0.05f, -0.002f, 0.001f, 0.f, 0.f, 0.f, 0.f};
        float* d_rows = upload(rows);
        float* d_radii2 = device_zeros<float>(N);
        DeviceVector<float> radii2(ttv(d_radii2, {N, 1}));
        auto dout = projection_3dgs_forward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "OPENCV",
                                            ttv(d_rows, {(int64_t)C, kCameraDistortionParams}), radii2, std::nullopt, std::nullopt, 0, 32, 0);
        backend::device_synchronize();
        float *q_aabb = device_zeros<float>(m * 4), *q_depths = device_zeros<float>(m), *q_radii = device_zeros<float>(N);
        float *q_xy = device_zeros<float>(m * 2), *q_depth = device_zeros<float>(m), *q_conic = device_zeros<float>(m * 3), *q_opac = device_zeros<float>(m),
              *q_rgb = device_zeros<float>(m * 3);
        if (ref_fwd_dist(0, 1, C, (uint32_t)N, W, H, d_means, d_quats, d_scales, d_opac, d_dc, d_sh, d_vm, d_intr, d_rows, q_aabb, q_depths, q_radii, q_xy, q_depth,
                         q_conic, q_opac, q_rgb) != 0) { std::fprintf(stderr, "ref_project_fwd_dist failed\n"); return 2; }
        auto ga = download((const float*)std::get<0>(dout).data_ptr(), m * 4), ra = download(q_aabb, m * 4), r0 = download(r_aabb, m * 4);
        std::vector<char> both(m);
        int64_t n_ref = 0, n_diff = 0, n_moved = 0;
        for (int64_t i = 0; i < m; ++i) {
            const bool kr = ra[4 * i + 2] > ra[4 * i], kg = ga[4 * i + 2] > ga[4 * i], k0 = r0[4 * i + 2] > r0[4 * i];
            n_ref += kr; n_diff += kr != kg; both[i] = kr && kg; n_moved += kr != k0;
        }
        report("distorted projection: visible set", n_ref > 500 && n_moved > 0 && (double)n_diff / (double)m <= 2e-3, (double)n_ref, (double)n_moved);
        auto& d_screen_out = std::get<2>(dout);
        report("distorted projection: xy", frac_bad(download(d_screen_out[0].data_ptr(), m * 2), download(q_xy, m * 2), 5e-3, 5e-4, &both, 2) <= 2e-3);
        report("distorted projection: conic", frac_bad(download(d_screen_out[2].data_ptr(), m * 3), download(q_conic, m * 3), 5e-3, 5e-4, &both, 3) <= 2e-3);
    }
    (void)v_w; (void)aw_out;

    // ---- 6. the live-tile map, and the intersection that uses it
    {
        typedef int (*RefTileActive)(const bool*, int, int, int, int, int, int32_t*);
        typedef int (*RefIntersectLive)(uint32_t, uint32_t, uint32_t, uint32_t, const float*, const float*, const float*, const float*, const float*,
                                        const int32_t*, int64_t*, int64_t*, int64_t, int64_t*, int64_t*, int32_t*, int32_t*, int32_t*, int64_t*, int32_t*);
        auto ref_tile_active = (RefTileActive)dlsym(ref, "ref_tile_active");
        auto ref_isect_live = (RefIntersectLive)dlsym(ref, "ref_intersect_tile_live");
        if (!ref_tile_active || !ref_isect_live) { std::fprintf(stderr, "missing live-tile entry points\n"); return 2; }
        std::vector<unsigned char> mask((size_t)C * H * W, 1);
        for (uint32_t c = 0; c < C; ++c)
            for (uint32_t y = 0; y < H; ++y)
                for (uint32_t x = W / 2; x < W; ++x) mask[((size_t)c * H + y) * W + x] = (y == H / 3 && x == W - 3) ? 1 : 0;
        unsigned char* d_mask = upload(mask);
        const int64_t n_tiles = (int64_t)C * th * tw;
        int32_t* live_a = device_zeros<int32_t>(n_tiles);
        int32_t* live_r = device_zeros<int32_t>(n_tiles);
        compute_tile_active(std::make_tuple((uint64_t)d_mask, (uint32_t)1, std::vector<int64_t>{(int64_t)C, (int64_t)H, (int64_t)W}), (int)C, (int)W, (int)H, live_a);
        if (ref_tile_active((const bool*)d_mask, (int)C, (int)H, (int)W, (int)W, (int)H, live_r) != 0) return 2;
        auto la = download(live_a, n_tiles), lr = download(live_r, n_tiles);
        int64_t n_live = 0;
        for (auto v : lr) n_live += v;
        report("live-tile map", la == lr && n_live > 0 && n_live < n_tiles, (double)n_live, (double)n_tiles);
        auto [ids2, flat2, offs2] = do_intersect_tile_generic(aabb_nd, depths_nd, &ref_screen[0], &ref_screen[2], &ref_screen[3], C,
                                                              ttv(d_intr, {(int64_t)C, 4}), W, H, nullptr, live_a);
        int64_t M2 = 0; int32_t sel2 = 0;
        if (ref_isect_live(C, (uint32_t)N, W, H, r_aabb, r_depths, r_xy, r_conic, r_opac, live_r, r_tps, r_cum, cap, r_ids_a, r_ids_b, r_fl_a, r_fl_b, r_offs,
                           &M2, &sel2) != 0) return 2;
        report("live intersection: pair count", (int64_t)ids2.size() == M2 && M2 < M, (double)ids2.size(), (double)M2);
        report("live intersection: sorted keys", download(ids2.data_ptr(), M2) == download(sel2 ? r_ids_b : r_ids_a, M2));
        report("live intersection: flatten ids", download(flat2.data_ptr(), M2) == download(sel2 ? r_fl_b : r_fl_a, M2));
        report("live intersection: tile ranges", download(offs2.data_ptr(), n_tiles) == download(r_offs, n_tiles));
    }

    // ---- 7. the loss driver: two levels, a mask, the loss map of mode 1
    {
        typedef int (*RefLoss)(int, int, int, int, const float*, const float*, const bool*, int, int, float, float, int, float*, float*, float*, float*);
        auto ref_loss = (RefLoss)dlsym(ref, "ref_multi_scale_loss");
        if (!ref_loss) { std::fprintf(stderr, "missing ref_multi_scale_loss\n"); return 2; }
        const int64_t P = (int64_t)C * H * W;
        std::vector<float> img_a(P * 3), img_b(P * 3);
        for (auto& v : img_a) v = uf(0.f, 1.f);
        for (int64_t i = 0; i < P * 3; ++i) img_b[i] = std::min(1.0f, std::max(0.0f, img_a[i] + 0.2f * (uf(0.f, 1.f) - 0.5f)));
        std::vector<unsigned char> mask((size_t)P, 1);
        for (int64_t i = 0; i < P; ++i) mask[i] = (i % 7 == 3 || (i / W) % H < H / 5) ? 0 : 1;
        float *d_a = upload(img_a), *d_b = upload(img_b);
        unsigned char* d_mask = upload(mask);
        float *v_ours = device_zeros<float>(P * 3), *v_ref = device_zeros<float>(P * 3), *lm_ours = device_zeros<float>(P), *lm_ref = device_zeros<float>(P);
        std::array<float, (int)LossWeightIndex::length> weights{};
        weights[(int)LossWeightIndex::RgbSupL1] = 0.8f;
        PerPixelGrads grads{};
        grads.v_render_rgb = ttv(v_ours, {(int64_t)C, H, W, 3});
        TorchTensorView none((uint64_t)0, 4u, std::vector<int64_t>{0, 0, 0, 0});
        std::vector<bool> needs(13, false);
        needs[0] = true;
        LossValues lv = compute_multi_scale_per_pixel_losses(
            2, ttv(d_a, {(int64_t)C, H, W, 3}), ttv(d_b, {(int64_t)C, H, W, 3}), none, none, none, none, none, none, none, none, none, none, none,
            std::make_tuple((uint64_t)d_mask, (uint32_t)1, std::vector<int64_t>{(int64_t)C, (int64_t)H, (int64_t)W, 1}), true, weights, 0.2f, none, needs,
            (long)C, none, ttv(lm_ours, {(int64_t)C, H, W, 1}), 1, 0.9f, 0.0f, grads);
        float r_rgb_loss = 0.f, r_ssim = 0.f;
        if (ref_loss(2, (int)C, (int)H, (int)W, d_a, d_b, (const bool*)d_mask, (int)H, (int)W, 0.8f, 0.2f, 1, v_ref, lm_ref, &r_rgb_loss, &r_ssim) != 0) return 2;
        auto rv = download(v_ref, P * 3);
        report("loss driver: colour gradient", frac_bad(download(v_ours, P * 3), rv, 2e-6 * max_abs(rv), 2e-4) <= 1e-3, max_abs(rv));
        report("loss driver: loss map", frac_bad(download(lm_ours, P), download(lm_ref, P), 2e-5, 1e-4) <= 1e-3);
        report("loss driver: scalars", std::fabs(lv.rgb_loss - r_rgb_loss) <= 1e-5 * std::fabs(r_rgb_loss) + 1e-7 && std::fabs(lv.ssim - r_ssim) <= 2e-5,
               lv.rgb_loss, lv.ssim);
    }

    // ---- 8. the optimiser launch functions
    {
        typedef int (*RefGeo)(int64_t, int, float, int, float, float, float, float, float*, float*, float*, float*, float*, float*, float*, float*, float*,
                              float*, float*, float*, float*, float*, float*, float*);
        typedef int (*RefPlain)(int64_t, int, float, float, float, float, int, float*, float*, float*, float*);
        typedef int (*RefQQ)(int64_t, int, float, float, float, int, int, float*, uint8_t*, float*, uint8_t*, float*);
        auto ref_geo = (RefGeo)dlsym(ref, "ref_adam_geometry");
        auto ref_plain = (RefPlain)dlsym(ref, "ref_adam_plain");
        auto ref_qq = (RefQQ)dlsym(ref, "ref_adam_qq");
        if (!ref_geo || !ref_plain || !ref_qq) { std::fprintf(stderr, "missing optimiser entry points\n"); return 2; }
        auto noisy = [&](int64_t n, float scale, float shift) { std::vector<float> v(n); for (auto& x : v) x = shift + scale * (uf(0.f, 1.f) - 0.5f); return v; };
        const int widths[4] = {3, 4, 3, 1};
        float *p_o[4], *g_o[4], *a_o[4], *b_o[4], *p_r[4], *g_r[4], *a_r[4], *b_r[4];
        for (int k = 0; k < 4; ++k) {
            auto p = noisy(N * widths[k], 2.f, 0.f), g = noisy(N * widths[k], 1e-3f, 0.f), a = noisy(N * widths[k], 1e-4f, 0.f), b = noisy(N * widths[k], 1e-8f, 1e-8f);
            p_o[k] = upload(p); g_o[k] = upload(g); a_o[k] = upload(a); b_o[k] = upload(b);
            p_r[k] = upload(p); g_r[k] = upload(g); a_r[k] = upload(a); b_r[k] = upload(b);
        }
        auto dv3 = [&](float* p) { return DeviceVector<float3>(ttv(p, {N, 3})); };
        auto dv4 = [&](float* p) { return DeviceVector<float4>(ttv(p, {N, 4})); };
        auto dv1 = [&](float* p) { return DeviceVector<float>(ttv(p, {N, 1})); };
        fused_optim_3dgs_geometry(N, dv3(p_o[0]), dv3(g_o[0]), dv3(a_o[0]), dv3(b_o[0]), dv4(p_o[1]), dv4(g_o[1]), dv4(a_o[1]), dv4(b_o[1]), dv3(p_o[2]),
                                  dv3(g_o[2]), dv3(a_o[2]), dv3(b_o[2]), dv1(p_o[3]), dv1(g_o[3]), dv1(a_o[3]), dv1(b_o[3]), DeviceVector<float3>{},
                                  DeviceVector<float3>{}, DeviceVector<float>{}, DeviceVector<float>{}, 1e-3f, 2e-3f, 5e-3f, 5e-2f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f,
                                  0.f, 0.f, false, NonShQuantState{}, GradQuantBuffers{}, 7, DeviceVector<int32_t>{}, 0.25f, true);
        if (ref_geo(N, 7, 0.25f, 1, 1e-3f, 2e-3f, 5e-3f, 5e-2f, p_r[0], g_r[0], a_r[0], b_r[0], p_r[1], g_r[1], a_r[1], b_r[1], p_r[2], g_r[2], a_r[2], b_r[2],
                    p_r[3], g_r[3], a_r[3], b_r[3]) != 0) return 2;
        bool ok = true, zeroed = true;
        for (int k = 0; k < 4; ++k) {
            ok = ok && frac_bad(download(p_o[k], N * widths[k]), download(p_r[k], N * widths[k]), 1e-6, 1e-4) <= 1e-3;
            ok = ok && frac_bad(download(a_o[k], N * widths[k]), download(a_r[k], N * widths[k]), 1e-9, 1e-4) <= 1e-3;
            zeroed = zeroed && max_abs(download(g_o[k], N * widths[k])) == 0.f;
        }
        report("fused_optim_3dgs_geometry", ok && zeroed);
        // the same function with the moments of all five arrays in 16-bit codes, two steps from the zero state
        {
            typedef int (*RefQ16)(int64_t, int, float, int, float, float, float, float, float, float, float*, float*, float*, float*, float*, float*, float*, float*,
                                  float*, float*, uint8_t* const*, float* const*, const float*, const int32_t*);
            auto ref_q16 = (RefQ16)dlsym(ref, "ref_adam_geometry_q16");
            if (!ref_q16) { std::fprintf(stderr, "missing ref_adam_geometry_q16\n"); return 2; }
            const int w5[5] = {3, 4, 3, 1, 3};
            const double lr5[5] = {1e-3, 2e-3, 5e-3, 5e-2, 2.5e-3};
            const int64_t blocks = (N + 255) / 256;
            float *po[5], *go[5], *pr[5], *gr[5], *bo[5], *br[5];
            uint8_t *qo[5], *qr[5];
            for (int k = 0; k < 5; ++k) {
                auto p = noisy(N * w5[k], 2.f, 0.f);
                po[k] = upload(p); pr[k] = upload(p);
                std::vector<uint8_t> zq(N * w5[k] * 4, 0); std::vector<float> zb(blocks * 4, 0.f);
                qo[k] = upload(zq); qr[k] = upload(zq); bo[k] = upload(zb); br[k] = upload(zb);
            }
            bool okq = true, okb = true;      // parameters; bounds of the codes
            int64_t worst = 0, far = 0, n_codes = 0;   // largest difference of the decoded moments in quanta, and how many beyond 4: the second step starts from each side's own codes
            for (int step = 1; step <= 2; ++step) {
                for (int k = 0; k < 5; ++k) { auto g = noisy(N * w5[k], 1e-3f, 0.f); go[k] = upload(g); gr[k] = upload(g); }
                NonShQuantState nq;
                nq.enabled = true;
                nq.means_packed = qo[0]; nq.quats_packed = qo[1]; nq.scales_packed = qo[2]; nq.opacities_packed = qo[3]; nq.features_dc_packed = qo[4];
                nq.means_bounds = (float4*)bo[0]; nq.quats_bounds = (float4*)bo[1]; nq.scales_bounds = (float4*)bo[2]; nq.opacities_bounds = (float4*)bo[3];
                nq.features_dc_bounds = (float4*)bo[4];
                fused_optim_3dgs_geometry(N, dv3(po[0]), dv3(go[0]), DeviceVector<float3>{}, DeviceVector<float3>{}, dv4(po[1]), dv4(go[1]), DeviceVector<float4>{},
                                          DeviceVector<float4>{}, dv3(po[2]), dv3(go[2]), DeviceVector<float3>{}, DeviceVector<float3>{}, dv1(po[3]), dv1(go[3]),
                                          DeviceVector<float>{}, DeviceVector<float>{}, dv3(po[4]), dv3(go[4]), DeviceVector<float>{}, DeviceVector<float>{}, 1e-3f,
                                          2e-3f, 5e-3f, 5e-2f, 2.5e-3f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.05f, false, nq, GradQuantBuffers{}, step,
                                          DeviceVector<int32_t>{}, 0.25f, false);
                if (ref_q16(N, step, 0.25f, 0, 1e-3f, 2e-3f, 5e-3f, 5e-2f, 2.5e-3f, 0.05f, pr[0], gr[0], pr[1], gr[1], pr[2], gr[2], pr[3], gr[3], pr[4], gr[4], qr, br,
                            nullptr, nullptr) != 0) return 2;
                for (int k = 0; k < 5; ++k) {
                    okq = okq && frac_bad(download(po[k], N * w5[k]), download(pr[k], N * w5[k]), 1e-6 + 2e-3 * lr5[k], 1e-4) <= 1e-3;   // a code is worth ~1e-4 of a step
                    okb = okb && frac_bad(download(bo[k], blocks * 4), download(br[k], blocks * 4), 1e-5, 1e-3) == 0.0;
                    auto co = download((uint16_t*)qo[k], N * w5[k] * 2), cr = download((uint16_t*)qr[k], N * w5[k] * 2);
                    // codes are compared as the values they stand for: the lower log-s bound of a block is set by its smallest
                    // gradient entry, which for quaternions is what the tangent projection leaves of two nearly equal numbers, so
                    // the bound (and with it every code of the block) shifts with the arithmetic while the decoded moments do not
                    auto hb = download(bo[k], blocks * 4), hr = download(br[k], blocks * 4);
                    for (size_t i = 0; i < co.size(); ++i) {
                        const int64_t b = (int64_t)(i / 2) / (256 * w5[k]);
                        const int c = (int)(i & 1) * 2;       // 0: u bounds, 2: log-s bounds
                        const double qo_ = hb[4 * b + c] + (hb[4 * b + c + 1] - hb[4 * b + c]) * (co[i] / 65535.0);
                        const double qr_ = hr[4 * b + c] + (hr[4 * b + c + 1] - hr[4 * b + c]) * (cr[i] / 65535.0);
                        const double quantum = (hr[4 * b + c + 1] - hr[4 * b + c]) / 65535.0;
                        const double d = std::fabs(qo_ - qr_) / std::max(quantum, 1e-12);
                        worst = std::max(worst, (int64_t)std::ceil(d)); far += d > 4.0; ++n_codes;
                    }
                }
            }
            report("fused_optim_3dgs_geometry, 16-bit moments", okq && okb && worst <= 64 && far * 1000 <= n_codes, (double)worst, (double)far);
        }
        // plain Adam on a [N, 3] array with the DC offset
        auto p = noisy(N * 3, 6.f, 0.f), g = noisy(N * 3, 1e-3f, 0.f), a = noisy(N * 3, 1e-4f, 0.f), b = noisy(N * 3, 1e-8f, 1e-8f);
        float *po = upload(p), *go = upload(g), *ao = upload(a), *bo = upload(b), *pr = upload(p), *gr = upload(g), *ar = upload(a), *br = upload(b);
        auto nd = [&](float* q, int64_t w) { return DeviceTensorFloatND(ttv(q, {N, w, 1})); };
        fused_adam_step(N, nd(po, 3), nd(go, 3), nd(ao, 3), nd(bo, 3), 2.5e-3f, 5, DeviceVector<int32_t>{}, 0.3f, 0.5f / 0.28209479f, 0.5f, false);
        if (ref_plain(N * 3, 5, 2.5e-3f, 0.3f, 0.5f / 0.28209479f, 0.5f, 0, pr, gr, ar, br) != 0) return 2;
        report("fused_adam_step", frac_bad(download(po, N * 3), download(pr, N * 3), 1e-6, 1e-4) <= 1e-3 &&
                                  frac_bad(download(bo, N * 3), download(br, N * 3), 1e-12, 1e-4) <= 1e-3);
        // quantised values + quantised state
        const int64_t cells = N * 45, blocks = (cells + 255) / 256;
        auto sh = noisy(cells, 0.4f, 0.f), gsh = noisy(cells, 1e-3f, 0.f);
        std::vector<uint16_t> codes(cells);
        std::vector<float> vb(blocks * 2), ob(blocks * 4);
        for (int64_t bl = 0; bl < blocks; ++bl) {
            float lo = 1e30f, hi = -1e30f;
            for (int64_t i = bl * 256; i < std::min(cells, bl * 256 + 256); ++i) { lo = std::min(lo, sh[i]); hi = std::max(hi, sh[i]); }
            vb[2 * bl] = lo; vb[2 * bl + 1] = hi;
            for (int64_t i = bl * 256; i < std::min(cells, bl * 256 + 256); ++i) codes[i] = (uint16_t)std::lround(65535.0 * (sh[i] - lo) / std::max(hi - lo, 1e-30f));
            ob[4 * bl] = -0.5f; ob[4 * bl + 1] = 0.5f; ob[4 * bl + 2] = 0.f; ob[4 * bl + 3] = 25.f;
        }
        std::vector<uint8_t> state(cells * 2);
        for (auto& v : state) v = (uint8_t)(uf(0.f, 1.f) * 255.f);
        float *gq_o = upload(gsh), *gq_r = upload(gsh), *vb_o = upload(vb), *vb_r = upload(vb), *ob_o = upload(ob), *ob_r = upload(ob);
        uint16_t *c_o = upload(codes), *c_r = upload(codes);
        uint8_t *s_o = upload(state), *s_r = upload(state);
        fused_adam_step_quantized_value(N, cells, nd(gq_o, 45), nullptr, nullptr, s_o, (float4*)ob_o, (uint8_t*)c_o, (float2*)vb_o, 2.5e-3f, 3, DeviceVector<int32_t>{},
                                        0.f, 0.f, 8, 16, 0.5f, false);
        if (ref_qq(cells, 3, 2.5e-3f, 0.f, 0.5f, 0, 16, gq_r, s_r, ob_r, (uint8_t*)c_r, vb_r) != 0) return 2;
        auto co = download(c_o, cells), cr = download(c_r, cells);
        int64_t off = 0;
        for (int64_t i = 0; i < cells; ++i) off += std::abs((int)co[i] - (int)cr[i]) > 1;
        report("fused_adam_step_quantized_value", off <= cells / 1000 && frac_bad(download(vb_o, blocks * 2), download(vb_r, blocks * 2), 1e-7, 1e-5) <= 1e-3, (double)off);
    }
    std::printf(g_failures ? "adapter_parity: %d check(s) FAILED\n" : "adapter_parity: all checks passed\n", g_failures);
    return g_failures ? 1 : 0;
}
