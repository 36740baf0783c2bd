// Parity driver for the adapter: calls the reference's kernel-launch functions -- through the reference's own
// declarations and tensor types, exactly as src/engine and the reference's parity tools do
// (src/backend/tests/render_parity.cpp:196-300, raster_bwd_parity.cpp:190-325) -- with ssb_adapter.cu supplying their
// definitions, and holds every output against the reference's own kernels run on the same inputs (the launch shims of the
// reference-side library, loaded at run time).  Stage by stage, each stage fed the reference's upstream outputs; tolerances
// are the reference tools' model |d| <= atol + rtol |ref| with a capped violation fraction.
//
//   adapter_parity <path to libssb_ref.so>        exit code 0 = every check passed
#include <kernels/projection/ProjectionFwd.cuh>
#include <kernels/raster/RasterizationBwd.cuh>
#include <kernels/raster/RasterizationFwd.cuh>
#include <kernels/tile/IntersectTile.cuh>

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
    // ---- 5. what the library does not cover is refused the way the reference refuses bad arguments
    bool threw = false;
    try {
        projection_3dgs_forward(N, 3, in_splats, ttv(d_vm, {(int64_t)C, 16}), ttv(d_intr, {(int64_t)C, 4}), W, H, "PINHOLE", "OPENCV",
                                ttv(nullptr, {(int64_t)C, kCameraDistortionParams}), radii, std::nullopt, std::nullopt, 0, 32, 0);
    } catch (const std::runtime_error&) { threw = true; }
    report("unsupported distortion tier throws", threw);
    (void)v_w; (void)aw_out;
    std::printf(g_failures ? "adapter_parity: %d check(s) FAILED\n" : "adapter_parity: all checks passed\n", g_failures);
    return g_failures ? 1 : 0;
}
