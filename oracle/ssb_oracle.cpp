// TEST INFRASTRUCTURE -- NOT PRODUCT CODE.
//
// CPU restatement (C++17 + OpenMP) of one 3D-Gaussian-splatting training
// iteration as implemented by spirula-studio's CUDA backend.  It exists only
// to check the CUDA library (tests, the smoke check) and to be timed as the
// CPU baseline by bench.py.  Nothing in the shipped library calls into this
// file.  Every function cites the reference file:line it restates.
//
// PARITY PIN STATUS: pinned.  The reference tree holds no golden vectors for this
// path (its parity tools dump-then-compare against a CUDA build made on the spot)
// and has no CPU implementation, so the pins are outputs of the reference's OWN
// device code: oracle/Makefile.ref compiles the reference's kernels from the
// sources where they lie into oracle/_ref/libssb_ref.so, tests/golden/make_golden.py
// runs them on a B200 on seeded scenes, and tests/test_golden_cpu.py compares every
// function below, stage by stage, with those fixtures (tests/golden/*.npz) under
// the reference parity tools' tolerance model.  In addition the backward passes
// are checked against central finite differences of the forward passes, and the
// integer stages against std::stable_sort / brute-force definitions.
//
// Numerics: plain IEEE fp32, compiled with -ffp-contract=off so that no FMA is
// formed behind the source.  The integer-producing stage (tile counting and key
// generation) is written as an explicit sequence of single fp32 operations and
// a polynomial logarithm, so a GPU kernel that performs the same sequence with
// round-to-nearest intrinsics reproduces its integers bit for bit.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <numeric>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr float ALPHA_THRESHOLD = 1.0f / 255.0f;   // src/core/Common.cuh:45
constexpr int TILE = 16;                           // TILE_SIZE_X * MACRO_TILE_SIZE_X, src/core/Common.cuh:36-39
constexpr int MICRO = 8;                           // TILE_SIZE_X, src/core/Common.cuh:36
constexpr int NUM_SH = 15;                         // degree 3: src/primitives/PrimitiveBase3DGS.cuh:30-32

enum CameraModel { PINHOLE = 0, FISHEYE = 1, EQUISOLID = 2, EQUIRECT = 3 };  // src/core/Common.cuh:96-101

// ---------------------------------------------------------------------------
// Forward-mode dual numbers with K tangent lanes.  Used to obtain the exact
// Jacobian of the projection, from which the vector-Jacobian product the
// reference gets from Slang's reverse-mode autodiff is formed.
// ---------------------------------------------------------------------------
template <int K>
struct Dual {
    float v;
    float d[K];
    Dual() : v(0.f) { for (int i = 0; i < K; ++i) d[i] = 0.f; }
    Dual(float x) : v(x) { for (int i = 0; i < K; ++i) d[i] = 0.f; }
};
template <int K> inline Dual<K> operator+(const Dual<K>& a, const Dual<K>& b) { Dual<K> r; r.v = a.v + b.v; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] + b.d[i]; return r; }
template <int K> inline Dual<K> operator-(const Dual<K>& a, const Dual<K>& b) { Dual<K> r; r.v = a.v - b.v; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] - b.d[i]; return r; }
template <int K> inline Dual<K> operator-(const Dual<K>& a) { Dual<K> r; r.v = -a.v; for (int i = 0; i < K; ++i) r.d[i] = -a.d[i]; return r; }
template <int K> inline Dual<K> operator*(const Dual<K>& a, const Dual<K>& b) { Dual<K> r; r.v = a.v * b.v; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * b.v + a.v * b.d[i]; return r; }
template <int K> inline Dual<K> operator/(const Dual<K>& a, const Dual<K>& b) { Dual<K> r; float ib = 1.0f / b.v; r.v = a.v * ib; for (int i = 0; i < K; ++i) r.d[i] = (a.d[i] - r.v * b.d[i]) * ib; return r; }
template <int K> inline Dual<K> operator+(const Dual<K>& a, float b) { Dual<K> r = a; r.v += b; return r; }
template <int K> inline Dual<K> operator+(float b, const Dual<K>& a) { Dual<K> r = a; r.v += b; return r; }
template <int K> inline Dual<K> operator-(const Dual<K>& a, float b) { Dual<K> r = a; r.v -= b; return r; }
template <int K> inline Dual<K> operator-(float b, const Dual<K>& a) { Dual<K> r = -a; r.v += b; return r; }
template <int K> inline Dual<K> operator*(const Dual<K>& a, float b) { Dual<K> r; r.v = a.v * b; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * b; return r; }
template <int K> inline Dual<K> operator*(float b, const Dual<K>& a) { return a * b; }
template <int K> inline Dual<K> operator/(const Dual<K>& a, float b) { return a * (1.0f / b); }
template <int K> inline Dual<K> operator/(float a, const Dual<K>& b) { return Dual<K>(a) / b; }
template <int K> inline Dual<K> d_sqrt(const Dual<K>& a) { Dual<K> r; r.v = std::sqrt(a.v); float s = 0.5f / r.v; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * s; return r; }
template <int K> inline Dual<K> d_exp(const Dual<K>& a) { Dual<K> r; r.v = std::exp(a.v); for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * r.v; return r; }
template <int K> inline Dual<K> d_log(const Dual<K>& a) { Dual<K> r; r.v = std::log(a.v); float s = 1.0f / a.v; for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * s; return r; }
template <int K> inline Dual<K> d_sin(const Dual<K>& a) { Dual<K> r; r.v = std::sin(a.v); float c = std::cos(a.v); for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * c; return r; }
template <int K> inline Dual<K> d_cos(const Dual<K>& a) { Dual<K> r; r.v = std::cos(a.v); float s = -std::sin(a.v); for (int i = 0; i < K; ++i) r.d[i] = a.d[i] * s; return r; }
template <int K> inline Dual<K> d_atan2(const Dual<K>& y, const Dual<K>& x) { Dual<K> r; r.v = std::atan2(y.v, x.v); float den = 1.0f / (x.v * x.v + y.v * y.v); for (int i = 0; i < K; ++i) r.d[i] = (x.v * y.d[i] - y.v * x.d[i]) * den; return r; }
inline float d_sqrt(float a) { return std::sqrt(a); }
inline float d_exp(float a) { return std::exp(a); }
inline float d_log(float a) { return std::log(a); }
inline float d_sin(float a) { return std::sin(a); }
inline float d_cos(float a) { return std::cos(a); }
inline float d_atan2(float y, float x) { return std::atan2(y, x); }
inline float val(float a) { return a; }
template <int K> inline float val(const Dual<K>& a) { return a.v; }
// clamp whose derivative follows whichever argument is selected; the interior
// (bounds included) selects x.  Same selection rule as Slang's clamp
// derivative (src/generated/primitive_3dgs.cuh:307-353).
template <class S> inline S d_clamp(const S& x, const S& lo, const S& hi) {
    if (val(x) < val(lo)) return lo;
    if (val(x) > val(hi)) return hi;
    return x;
}

struct Camera {
    float R[9];
    float t[3];
    float fx, fy, cx, cy;
    int W, H;
    int model;
    int n_sh = 15;           // SH coefficients past DC in use: (degree + 1)^2 - 1 of the active degree (Vanilla3DGS<degree>)
    int dist = 0;            // CameraDistortionType: 0 none, 1 OpenCV, 2 thin prism, 3 rational (src/core/Common.cuh)
    float coeffs[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
};

inline Camera load_camera(const float* viewmats, const float* intrins, int cid, int W, int H, int model, int dist = 0,
                          const float* dist_coeffs = nullptr) {
    // src/kernels/projection/ProjectionFwd_kernel.cuh:50-59: rows 0..2 of the
    // row-major 4x4 world-to-camera matrix are [R | t].
    const float* m = viewmats + 16 * cid;
    Camera c;
    c.R[0] = m[0]; c.R[1] = m[1]; c.R[2] = m[2];
    c.R[3] = m[4]; c.R[4] = m[5]; c.R[5] = m[6];
    c.R[6] = m[8]; c.R[7] = m[9]; c.R[8] = m[10];
    c.t[0] = m[3]; c.t[1] = m[7]; c.t[2] = m[11];
    c.fx = intrins[4 * cid + 0]; c.fy = intrins[4 * cid + 1];
    c.cx = intrins[4 * cid + 2]; c.cy = intrins[4 * cid + 3];
    c.W = W; c.H = H; c.model = model;
    c.dist = dist;
    // CameraDistortionCoeffsBuffer::load (src/core/Common.cuh:152-169): rows of eight floats; a null buffer reads as zeros
    if (dist != 0 && dist_coeffs) for (int i = 0; i < 8; ++i) c.coeffs[i] = dist_coeffs[8 * cid + i];
    return c;
}

template <class S>
struct ProjResult {
    S mean2d[2];
    S depth;
    S conic[3];
    S opacity;
    float aabb[4];
    float sorting_depth;
    float radius;
};

// src/shaders/projection_utils.slang:1012-1029
inline float get_sorting_depth(int model, const float p[3]) {
    if (model == PINHOLE) return p[2];
    if (model == EQUIRECT) return p[0] * p[0] + p[1] * p[1] + p[2] * p[2];
    float x = p[0], y = p[1], z = p[2];
    return z * z * z * z + (1.0f / 512.0f) * (x * x + y * y) * (x * x + y * y);
}

// src/shaders/projection_utils.slang:1033-1043
inline float view_radius_3dgs(const float mean[3], const float log_scale[3], float logit_opacity, const float campos[3]) {
    float extend = std::sqrt(2.0f * std::log(std::max(255.0f / (1.0f + std::exp(-logit_opacity)), 1.0f)));
    float radius = std::exp(std::max(log_scale[0], std::max(log_scale[1], log_scale[2]))) * extend;
    float dx = mean[0] - campos[0], dy = mean[1] - campos[1], dz = mean[2] - campos[2];
    float dist = std::sqrt(dx * dx + dy * dy + dz * dz);
    return radius / (std::max(dist, radius) + std::sqrt(std::max(dist * dist - radius * radius, 0.0f)));
}

// ---- lens distortion tiers (src/shaders/projection_utils.slang:208-298) -------------------------------------------
// A value over S with its two partial derivatives with respect to the undistorted coordinates (u, v).  The reference
// takes the 2x2 Jacobian of a tier by forward-mode autodiff of the tier's formula (camera_distortion_jac, :300-308);
// evaluating the formula in this arithmetic is the same thing, and with S itself a dual number the Jacobian carries
// its own derivatives with respect to the splat.
template <class S> struct Jet2 { S v, du, dv; };
template <class S> inline Jet2<S> operator+(const Jet2<S>& a, const Jet2<S>& b) { return {a.v + b.v, a.du + b.du, a.dv + b.dv}; }
template <class S> inline Jet2<S> operator*(const Jet2<S>& a, const Jet2<S>& b) { return {a.v * b.v, a.du * b.v + a.v * b.du, a.dv * b.v + a.v * b.dv}; }
template <class S> inline Jet2<S> operator/(const Jet2<S>& a, const Jet2<S>& b) {
    S q = a.v / b.v;
    return {q, (a.du - q * b.du) / b.v, (a.dv - q * b.dv) / b.v};
}
template <class S> inline Jet2<S> operator+(float a, const Jet2<S>& b) { return {a + b.v, b.du, b.dv}; }
template <class S> inline Jet2<S> operator*(float a, const Jet2<S>& b) { return {a * b.v, a * b.du, a * b.dv}; }

// distort(uv) of one tier; coefficient order is the tier's own (:246 k1 k2 p1 p2; :262 k1 k2 k3 k4 p1 p2 sx1 sy1;
// :283 k1 k2 k3 k4 k5 k6 p1 p2 with k4..k6 in the denominator)
template <class T>
inline void distort_tier(int dist, const float* c, const T& u, const T& v, T& ou, T& ov) {
    T r2 = u * u + v * v;
    if (dist == 1) {
        float k1 = c[0], k2 = c[1], p1 = c[2], p2 = c[3];
        T radial = 1.0f + r2 * (k1 + k2 * r2);
        ou = u * radial + ((2.0f * p1) * (u * v) + p2 * (r2 + 2.0f * (u * u)));
        ov = v * radial + ((2.0f * p2) * (u * v) + p1 * (r2 + 2.0f * (v * v)));
    } else if (dist == 2) {
        float k1 = c[0], k2 = c[1], k3 = c[2], k4 = c[3], p1 = c[4], p2 = c[5], sx1 = c[6], sy1 = c[7];
        T radial = 1.0f + r2 * (k1 + r2 * (k2 + r2 * (k3 + k4 * r2)));
        ou = u * radial + (((2.0f * p1) * (u * v) + p2 * (r2 + 2.0f * (u * u))) + sx1 * r2);
        ov = v * radial + (((2.0f * p2) * (u * v) + p1 * (r2 + 2.0f * (v * v))) + sy1 * r2);
    } else {
        float k1 = c[0], k2 = c[1], k3 = c[2], k4 = c[3], k5 = c[4], k6 = c[5], p1 = c[6], p2 = c[7];
        T radial = (1.0f + r2 * (k1 + r2 * (k2 + k3 * r2))) / (1.0f + r2 * (k4 + r2 * (k5 + k6 * r2)));
        ou = u * radial + ((2.0f * p1) * (u * v) + p2 * (r2 + 2.0f * (u * u)));
        ov = v * radial + ((2.0f * p2) * (u * v) + p1 * (r2 + 2.0f * (v * v)));
    }
}

// Distorted coordinates and the Jacobian Dj = d(distort)/d(u, v), row major
template <class S>
inline void distort_with_jac(int dist, const float* c, const S& u, const S& v, S out[2], S Dj[4]) {
    Jet2<S> ju{u, S(1.f), S(0.f)}, jv{v, S(0.f), S(1.f)}, ou, ov;
    distort_tier<Jet2<S>>(dist, c, ju, jv, ou, ov);
    out[0] = ou.v; out[1] = ov.v;
    Dj[0] = ou.du; Dj[1] = ou.dv; Dj[2] = ov.du; Dj[3] = ov.dv;
}

// is_valid_distortion (:311-323): the map must stay a moderate, orientation-preserving stretch at uv
inline bool distortion_valid(int dist, const float* c, float u, float v) {
    float out[2], Dj[4];
    distort_with_jac<float>(dist, c, u, v, out, Dj);
    float jdet = std::min(Dj[0] * Dj[3] - Dj[1] * Dj[2], std::min(Dj[0], Dj[3]));
    return jdet > 0.25f && jdet < 4.0f && (u * out[0] + v * out[1]) >= 0.0f;
}

// Camera-model mean projection and its 2x3 Jacobian, both in S arithmetic.
// The reference obtains J by forward-mode autodiff of the same projection
// (src/shaders/projection_utils.slang:331-375 pinhole, :379-384,463-476
// fisheye, :505-518,537-548 equirectangular); the closed forms below are those
// derivatives written out.  Distortion tier "none" only.
template <class S>
inline void project_mean(int model, const S p[3], float fx, float fy, float cx, float cy, S uv[2], S J[6]) {
    if (model == PINHOLE) {
        S rz = 1.0f / p[2];
        S u = p[0] * rz, v = p[1] * rz;
        uv[0] = fx * u + cx;
        uv[1] = fy * v + cy;
        J[0] = fx * rz; J[1] = S(0.f); J[2] = -(fx * u) * rz;
        J[3] = S(0.f); J[4] = fy * rz; J[5] = -(fy * v) * rz;
    } else if (model == FISHEYE) {
        S r2 = p[0] * p[0] + p[1] * p[1];
        S r = d_sqrt(r2);
        S theta = d_atan2(r, p[2]);
        S rho2 = r2 + p[2] * p[2];
        if (val(theta) < 1e-3f) {
            // k = (1 - theta^2/3)/z, src/shaders/projection_utils.slang:382
            S k = (1.0f - theta * theta / 3.0f) / p[2];
            uv[0] = fx * (p[0] * k) + cx;
            uv[1] = fy * (p[1] * k) + cy;
            // d theta / d(x,y,z) = (z x / (r rho2), z y / (r rho2), -r / rho2);
            // near the axis r -> 0 and theta ~ r/z, so d theta/dx ~ x/(r z).
            // dk/dq = -(2 theta / 3) dtheta/dq / z  (q = x, y);  dk/dz adds -k/z.
            S rinv = (val(r) > 0.f) ? (1.0f / r) : S(0.f);
            S dtx = p[2] * p[0] * rinv / rho2, dty = p[2] * p[1] * rinv / rho2, dtz = -r / rho2;
            S c = -(2.0f / 3.0f) * theta / p[2];
            S dkx = c * dtx, dky = c * dty, dkz = c * dtz - k / p[2];
            J[0] = fx * (k + p[0] * dkx); J[1] = fx * (p[0] * dky); J[2] = fx * (p[0] * dkz);
            J[3] = fy * (p[1] * dkx); J[4] = fy * (k + p[1] * dky); J[5] = fy * (p[1] * dkz);
        } else {
            S k = theta / r;
            uv[0] = fx * (p[0] * k) + cx;
            uv[1] = fy * (p[1] * k) + cy;
            S dtx = p[2] * p[0] / (r * rho2), dty = p[2] * p[1] / (r * rho2), dtz = -r / rho2;
            // dk/dx = dtheta/dx / r - theta x / r^3
            S ir = 1.0f / r;
            S dkx = dtx * ir - theta * p[0] * ir * ir * ir;
            S dky = dty * ir - theta * p[1] * ir * ir * ir;
            S dkz = dtz * ir;
            J[0] = fx * (k + p[0] * dkx); J[1] = fx * (p[0] * dky); J[2] = fx * (p[0] * dkz);
            J[3] = fy * (p[1] * dkx); J[4] = fy * (k + p[1] * dky); J[5] = fy * (p[1] * dkz);
        }
    } else if (model == EQUISOLID) {
        // k = 2 sin(theta / 2) / r with theta = atan2(r, z) (src/shaders/projection_utils.slang:388-395; Jacobian by
        // forward-mode autodiff, :480-493).  With rho = |p|: sin(theta/2) = r / (2 rho cos(theta/2)) and
        // cos^2(theta/2) = (rho + z) / (2 rho), so k = sqrt(2 / (rho (rho + z))): the same function without the
        // cancellation of cos(theta/2) dtheta/r - 2 sin(theta/2)/r^2, and it contains the reference's series
        // (1 - theta^2/24)/z for r < 1e-6.  Behind the camera rho + z is taken as r^2 / (rho - z).
        S r2 = p[0] * p[0] + p[1] * p[1];
        S rho2 = r2 + p[2] * p[2];
        S rho = d_sqrt(rho2);
        S w = (val(p[2]) >= 0.f) ? (rho + p[2]) : (r2 / (rho - p[2]));
        S q = rho * w;
        S k = d_sqrt(2.0f / q);
        S c = -(k / (2.0f * q * rho));
        S dkx = c * (p[0] * (2.0f * rho + p[2]));
        S dky = c * (p[1] * (2.0f * rho + p[2]));
        S dkz = -(k * w / (2.0f * rho2));
        uv[0] = fx * (p[0] * k) + cx;
        uv[1] = fy * (p[1] * k) + cy;
        J[0] = fx * (k + p[0] * dkx); J[1] = fx * (p[0] * dky); J[2] = fx * (p[0] * dkz);
        J[3] = fy * (p[1] * dkx); J[4] = fy * (k + p[1] * dky); J[5] = fy * (p[1] * dkz);
    } else {  // EQUIRECT: lon = atan2(x, z), lat = atan2(y, hypot(x, z))
        S h2 = p[0] * p[0] + p[2] * p[2];
        S h = d_sqrt(h2);
        S lon = d_atan2(p[0], p[2]);
        S lat = d_atan2(p[1], h);
        uv[0] = fx * lon + cx;
        uv[1] = fy * lat + cy;
        S rho2 = h2 + p[1] * p[1];
        J[0] = fx * (p[2] / h2); J[1] = S(0.f); J[2] = fx * (-(p[0] / h2));
        J[3] = fy * (-(p[1] * p[0]) / (h * rho2)); J[4] = fy * (h / rho2); J[5] = fy * (-(p[1] * p[2]) / (h * rho2));
    }
}

// The same with a lens distortion tier between the camera model's normalised coordinates and the pixel grid
// (persp_proj_uv / fisheye_proj_uv / equisolid_proj_uv, src/shaders/projection_utils.slang:330-343,412-424,443-455, and
// their Jacobians by forward-mode autodiff, :363-375,463-493): uv = f * distort(n(p)) + c, J = diag(f) Dj dn/dp.
// `valid` (may be null) receives is_valid_distortion at n(p).
template <class S>
inline void project_mean_distorted(const Camera& cam, const S p[3], S uv[2], S J[6], bool* valid) {
    S n[2], Jn[6];
    project_mean<S>(cam.model, p, 1.0f, 1.0f, 0.0f, 0.0f, n, Jn);
    if (valid) *valid = distortion_valid(cam.dist, cam.coeffs, val(n[0]), val(n[1]));
    S d[2], Dj[4];
    distort_with_jac<S>(cam.dist, cam.coeffs, n[0], n[1], d, Dj);
    uv[0] = cam.fx * d[0] + cam.cx;
    uv[1] = cam.fy * d[1] + cam.cy;
    for (int j = 0; j < 3; ++j) {
        J[j] = cam.fx * (Dj[0] * Jn[j] + Dj[1] * Jn[3 + j]);
        J[3 + j] = cam.fy * (Dj[2] * Jn[j] + Dj[3] * Jn[3 + j]);
    }
}

// src/shaders/primitive_3dgs.slang:419-578 (projection_3dgs<model, D,
// assume_valid, eval3d=false>).  Returns false where the reference returns with
// aabb = 0.  With assume_valid every cull is skipped, as in the backward pass
// (src/shaders/primitive_3dgs.slang:644-653).
template <class S>
inline bool projection_3dgs(
    const Camera& cam, bool antialiased, bool assume_valid,
    const S mean[3], const S quat[4], const S scale[3], const S& in_opacity,
    const float mean_f[3], const float scale_f[3], float in_opacity_f,
    ProjResult<S>& out) {
    for (int i = 0; i < 4; ++i) out.aabb[i] = 0.f;
    out.sorting_depth = 0.f; out.radius = 0.f;
    out.mean2d[0] = S(0.f); out.mean2d[1] = S(0.f);
    out.conic[0] = out.conic[1] = out.conic[2] = S(0.f);
    out.opacity = S(0.f);

    const float* R = cam.R;
    // posW2C, src/shaders/projection_utils.slang:92-99
    S mc[3];
    for (int i = 0; i < 3; ++i)
        mc[i] = R[3 * i + 0] * mean[0] + R[3 * i + 1] * mean[1] + R[3 * i + 2] * mean[2] + cam.t[i];
    S len = d_sqrt(mc[0] * mc[0] + mc[1] * mc[1] + mc[2] * mc[2]);
    out.depth = len;                                   // :439 ray depth
    float cull_z = (cam.model == PINHOLE) ? val(mc[2]) : val(len);
    if (!assume_valid && cull_z <= 0.0f) return false;  // :440-443

    out.opacity = 1.0f / (1.0f + d_exp(-in_opacity));  // :447

    // quat_scale_to_covar(normalize(quat), exp(scale)), :484;
    // src/shaders/projection_utils.slang:72-88,114-124
    S qn = d_sqrt(quat[0] * quat[0] + quat[1] * quat[1] + quat[2] * quat[2] + quat[3] * quat[3]);
    S w = quat[0] / qn, x = quat[1] / qn, y = quat[2] / qn, z = quat[3] / qn;
    S Rq[9] = {
        1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y),
        2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x),
        2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)};
    S s[3] = {d_exp(scale[0]), d_exp(scale[1]), d_exp(scale[2])};
    S M[9];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) M[3 * i + j] = Rq[3 * i + j] * s[j];
    S cov[9];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j)
        cov[3 * i + j] = M[3 * i + 0] * M[3 * j + 0] + M[3 * i + 1] * M[3 * j + 1] + M[3 * i + 2] * M[3 * j + 2];
    // covarW2C, src/shaders/projection_utils.slang:103-109
    S RC[9], covc[9];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j)
        RC[3 * i + j] = R[3 * i + 0] * cov[0 + j] + R[3 * i + 1] * cov[3 + j] + R[3 * i + 2] * cov[6 + j];
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j)
        covc[3 * i + j] = RC[3 * i + 0] * R[3 * j + 0] + RC[3 * i + 1] * R[3 * j + 1] + RC[3 * i + 2] * R[3 * j + 2];

    S J[6];
    if (cam.dist != 0) {
        bool dist_ok = true;
        project_mean_distorted<S>(cam, mc, out.mean2d, J, assume_valid ? nullptr : &dist_ok);
        if (!assume_valid && !dist_ok) return false;      // persp_proj / fisheye_proj / equisolid_proj, :346-358,427-441
    } else {
        project_mean<S>(cam.model, mc, cam.fx, cam.fy, cam.cx, cam.cy, out.mean2d, J);
    }
    if (cam.model == PINHOLE) {
        // persp_proj: z < 0 is invalid (src/shaders/projection_utils.slang:349-355)
        if (!assume_valid && val(mc[2]) < 0.0f) return false;
        // src/shaders/primitive_3dgs.slang:84-95.  Both rows are limited with the
        // X limits (lim_x_*), as the reference does.
        float width = (float)cam.W;
        float lim_x_pos = width + 0.3f * (0.5f * width);
        float lim_x_neg = 0.3f * (0.5f * width);
        S rz = 1.0f / mc[2];
        S max_Jxz = -(-lim_x_neg - cam.cx) * rz;
        S min_Jxz = -(lim_x_pos - cam.cx) * rz;
        S max_Jyz = -(-lim_x_neg - cam.cy) * rz;
        S min_Jyz = -(lim_x_pos - cam.cy) * rz;
        J[2] = d_clamp(J[2], min_Jxz, max_Jxz);
        J[5] = d_clamp(J[5], min_Jyz, max_Jyz);
    }
    // cov2d = J covc J^T
    S JC[6];
    for (int i = 0; i < 2; ++i) for (int j = 0; j < 3; ++j)
        JC[3 * i + j] = J[3 * i + 0] * covc[0 + j] + J[3 * i + 1] * covc[3 + j] + J[3 * i + 2] * covc[6 + j];
    S c00 = JC[0] * J[0] + JC[1] * J[1] + JC[2] * J[2];
    S c01 = JC[0] * J[3] + JC[1] * J[4] + JC[2] * J[5];
    S c10 = JC[3] * J[0] + JC[4] * J[1] + JC[5] * J[2];
    S c11 = JC[3] * J[3] + JC[4] * J[4] + JC[5] * J[5];

    if (!assume_valid && (cam.model == FISHEYE || cam.model == EQUISOLID)) {
        // src/shaders/primitive_3dgs.slang:515-521
        float a = val(c00), b = val(c01), c = val(c10), d = val(c11);
        float invdet = 1.0f / (a * d - b * c);
        float i00 = d * invdet, i01 = -b * invdet, i10 = -c * invdet, i11 = a * invdet;
        float mx = val(out.mean2d[0]) - cam.cx, my = val(out.mean2d[1]) - cam.cy;
        float q = (i00 * mx + i01 * my) * mx + (i10 * mx + i11 * my) * my;
        float opac = val(out.opacity) * std::exp(-0.5f * q);
        if (val(mc[2]) < 0.0f && opac > 1.0f / 255.0f) return false;
    }

    // add_blur, :398-405,528-534
    const float eps2d = antialiased ? 0.1f : 0.3f;
    S det_orig = c00 * c11 - c01 * c10;
    c00 = c00 + eps2d; c11 = c11 + eps2d;
    S det_blur = c00 * c11 - c01 * c10;
    if (!assume_valid && val(det_blur) <= 0.f) return false;
    // inverse, src/shaders/projection_utils.slang:166-174
    S invdet = 1.0f / (c00 * c11 - c01 * c10);
    S i00 = c11 * invdet, i01 = -c01 * invdet, i11 = c00 * invdet;

    float extend = 3.33f;
    if (antialiased) {
        float r = val(det_orig) / val(det_blur);
        if (r > 0.f) out.opacity = out.opacity * d_sqrt(det_orig / det_blur);
        else out.opacity = out.opacity * 0.f;
    }
    if (!assume_valid && val(out.opacity) < ALPHA_THRESHOLD) return false;  // :543-546
    extend = std::min(extend, std::sqrt(2.0f * std::log(val(out.opacity) / ALPHA_THRESHOLD)));  // :549

    float radius_x = extend * std::sqrt(val(c00));
    float radius_y = extend * std::sqrt(val(c11));
    float xmin = val(out.mean2d[0]) - radius_x, xmax = val(out.mean2d[0]) + radius_x;
    float ymin = val(out.mean2d[1]) - radius_y, ymax = val(out.mean2d[1]) + radius_y;
    if (!assume_valid && (xmax <= 0 || xmin >= (float)cam.W || ymax <= 0 || ymin >= (float)cam.H)) return false;  // :562-568

    out.aabb[0] = xmin; out.aabb[1] = ymin; out.aabb[2] = xmax; out.aabb[3] = ymax;
    float mcf[3] = {val(mc[0]), val(mc[1]), val(mc[2])};
    out.sorting_depth = get_sorting_depth(cam.model, mcf);
    out.conic[0] = i00; out.conic[1] = i01; out.conic[2] = i11;
    // campos = -R^T t, :576
    float campos[3];
    for (int j = 0; j < 3; ++j) campos[j] = -(R[0 + j] * cam.t[0] + R[3 + j] * cam.t[1] + R[6 + j] * cam.t[2]);
    out.radius = view_radius_3dgs(mean_f, scale_f, in_opacity_f, campos);
    return true;
}

// Real SH basis of degree <= 3 evaluated at a unit direction, bands 1..3
// (15 values); the DC band is the constant 0.2820947917738781.
// src/shaders/harmonics.slang:154-251
template <class S>
inline void sh_basis_deg3(const S& x, const S& y, const S& z, S b[NUM_SH]) {
    const float fTmp0A = 0.48860251190292f;
    b[0] = -fTmp0A * y; b[1] = fTmp0A * z; b[2] = -fTmp0A * x;
    S z2 = z * z;
    S fTmp0B = -1.092548430592079f * z;
    const float fTmp1A = 0.5462742152960395f;
    S fC1 = x * x - y * y;
    S fS1 = 2.f * x * y;
    b[3] = fTmp1A * fS1;                                   // pSH4
    b[4] = fTmp0B * y;                                     // pSH5
    b[5] = 0.9461746957575601f * z2 - 0.3153915652525201f; // pSH6
    b[6] = fTmp0B * x;                                     // pSH7
    b[7] = fTmp1A * fC1;                                   // pSH8
    S fTmp0C = -2.285228997322329f * z2 + 0.4570457994644658f;
    S fTmp1B = 1.445305721320277f * z;
    const float fTmp2A = -0.5900435899266435f;
    S fC2 = x * fC1 - y * fS1;
    S fS2 = x * fS1 + y * fC1;
    b[8] = fTmp2A * fS2;                                   // pSH9
    b[9] = fTmp1B * fS1;                                   // pSH10
    b[10] = fTmp0C * y;                                    // pSH11
    b[11] = z * (1.865881662950577f * z2 - 1.119528997770346f);  // pSH12
    b[12] = fTmp0C * x;                                    // pSH13
    b[13] = fTmp1B * fC1;                                  // pSH14
    b[14] = fTmp2A * fC2;                                  // pSH15
}

// SH value-quantisation decode, src/shaders/harmonics.slang:115-140 and
// src/core/Tensor.h:1366-1378 (QuantizedTensor<BITS,256>::decode_v).
struct ShStore {
    const float* sh_f32;       // [N][15][3] or null
    const uint8_t* packed;     // q8 / q16 codes or null
    const float* bounds;       // float2 per block
    int bits;                  // 32, 16, 8
    int64_t bounds_stride;     // cells per bound
};
inline float sh_load(const ShStore& st, int64_t gid, int j, int ch) {
    int64_t cell = (int64_t)3 * NUM_SH * gid + 3 * j + ch;
    if (st.bits == 32) return st.sh_f32[cell];
    const float* mm = st.bounds + 2 * (cell / st.bounds_stride);
    if (st.bits == 8) {
        const float inv = 1.0f / 255.0f;
        return mm[0] + (mm[1] - mm[0]) * ((float)st.packed[cell] * inv);
    }
    const float inv = 1.0f / 65535.0f;
    const uint16_t* p16 = reinterpret_cast<const uint16_t*>(st.packed);
    return mm[0] + (mm[1] - mm[0]) * ((float)p16[cell] * inv);
}

// src/shaders/harmonics.slang:145-149,1055-1066: colour = max(SH(viewdir)+0.5, 0),
// viewdir = mean + R^T t (unnormalised; normalised inside the SH evaluation).
template <class S>
inline void sh_to_color(const Camera& cam, const S mean[3], const float dc[3], const float sh[NUM_SH][3], S rgb_raw[3], S basis[NUM_SH]) {
    const float* R = cam.R;
    S dir[3];
    for (int j = 0; j < 3; ++j)
        dir[j] = mean[j] + (R[0 + j] * cam.t[0] + R[3 + j] * cam.t[1] + R[6 + j] * cam.t[2]);
    S inv = 1.0f / d_sqrt(dir[0] * dir[0] + dir[1] * dir[1] + dir[2] * dir[2]);
    S x = dir[0] * inv, y = dir[1] * inv, z = dir[2] * inv;
    sh_basis_deg3<S>(x, y, z, basis);
    // sh<degree>_to_color (src/primitives/Primitive3DGS.cuh:76-97): the bands above the active degree are not read
    for (int j = cam.n_sh; j < NUM_SH; ++j) basis[j] = S(0.f);
    for (int ch = 0; ch < 3; ++ch) {
        S c = S(0.2820947917738781f * dc[ch]);
        for (int j = 0; j < cam.n_sh; ++j) c = c + basis[j] * sh[j][ch];
        rgb_raw[ch] = c;
    }
}

// Polynomial natural logarithm made only of single fp32 operations, so that the
// tile-count stage is reproducible on any IEEE machine.  Argument reduction to
// m in (sqrt(1/2), sqrt(2)] followed by the Cephes single-precision series.
inline float det_logf(float xin) {
    uint32_t bits; std::memcpy(&bits, &xin, 4);
    int e = (int)((bits >> 23) & 255u) - 127;
    uint32_t mb = (bits & 0x007fffffu) | 0x3f800000u;
    float m; std::memcpy(&m, &mb, 4);
    if (m > 1.41421356f) { m = m * 0.5f; e += 1; }
    float f = m - 1.0f;
    float z = f * f;
    float p = 7.0376836292E-2f;
    p = p * f; p = p + -1.1514610310E-1f;
    p = p * f; p = p + 1.1676998740E-1f;
    p = p * f; p = p + -1.2420140846E-1f;
    p = p * f; p = p + 1.4249322787E-1f;
    p = p * f; p = p + -1.6668057665E-1f;
    p = p * f; p = p + 2.0000714765E-1f;
    p = p * f; p = p + -2.4999993993E-1f;
    p = p * f; p = p + 3.3333331174E-1f;
    float fe = (float)e;
    float y = f * z; y = y * p;
    float t = -2.12194440e-4f * fe; y = y + t;
    t = 0.5f * z; y = y - t;
    float r = f + y;
    t = 0.693359375f * fe; r = r + t;
    return r;
}

// float -> int with NaN -> 0 and saturation: what cvt.rzi.s32.f32 does.
inline int f2i(float v) {
    if (!(v == v)) return 0;
    if (v >= 2147483648.0f) return 2147483647;
    if (v <= -2147483648.0f) return (-2147483647 - 1);
    return (int)v;
}
template <class T> inline T clampT(T x, T a, T b) { return x < a ? a : (x > b ? b : x); }  // src/kernels/tile/IntersectTile.cu:30-32

// src/kernels/tile/IntersectTile.cu:34-53
inline void ellipse_range_bound(float a, float b, float c, float y0, float y1, float& x0, float& x1) {
    float ac = a * c, bb = b * b;
    float det = ac - bb;
    float q = c / det;
    float sq = std::sqrt(q);
    float nb = -b;
    float r = nb / c;
    float ym = r * sq;
    float v0 = clampT(-ym, y0, y1);
    float v1 = clampT(ym, y0, y1);
    float bv0 = nb * v0, bv1 = nb * v1;
    float inv_a = 1.0f / a;
    float t0 = c * v0; t0 = t0 * v0; t0 = t0 - 1.0f; t0 = a * t0;
    float d0 = bv0 * bv0; d0 = d0 - t0;
    float t1 = c * v1; t1 = t1 * v1; t1 = t1 - 1.0f; t1 = a * t1;
    float d1 = bv1 * bv1; d1 = d1 - t1;
    float e0 = bv0 - std::sqrt(d0);
    float e1 = bv1 + std::sqrt(d1);
    x0 = inv_a * e0;
    x1 = inv_a * e1;
}

struct TileSpan { int xmin, xmax, ymin, ymax; };

// Visits the tiles one splat touches in the reference's order
// (src/kernels/tile/IntersectTile.cu:55-101 counting, :200-247 emitting).
template <class F>
inline void for_each_tile(const float xy[2], float ca, float cb, float cc, const TileSpan& g, F&& fn) {
    if ((g.ymax - g.ymin) * TILE <= (g.xmax - g.xmin) * TILE) {
        for (int y = g.ymin; y < g.ymax; ++y) {
            float y0 = (float)(y * TILE) - xy[1];
            float y1 = y0 + (float)TILE;
            float bx0, bx1;
            ellipse_range_bound(ca, cb, cc, y0, y1, bx0, bx1);
            int x0 = f2i(std::floor((bx0 + xy[0]) / (float)TILE));
            int x1 = f2i(std::ceil((bx1 + xy[0]) / (float)TILE));
            x0 = clampT(x0, g.xmin, g.xmax);
            x1 = clampT(x1, g.xmin, g.xmax);
            for (int x = x0; x < x1; ++x) fn(x, y);
        }
    } else {
        for (int x = g.xmin; x < g.xmax; ++x) {
            float x0 = (float)(x * TILE) - xy[0];
            float x1 = x0 + (float)TILE;
            float by0, by1;
            ellipse_range_bound(cc, cb, ca, x0, x1, by0, by1);
            int y0 = f2i(std::floor((by0 + xy[1]) / (float)TILE));
            int y1 = f2i(std::ceil((by1 + xy[1]) / (float)TILE));
            y0 = clampT(y0, g.ymin, g.ymax);
            y1 = clampT(y1, g.ymin, g.ymax);
            for (int y = y0; y < y1; ++y) fn(x, y);
        }
    }
}

inline bool tile_setup(const float aabb[4], const float conic_in[3], float opac, int tw, int th, TileSpan& g, float conic[3]) {
    float xmin = aabb[0], ymin = aabb[1], xmax = aabb[2], ymax = aabb[3];
    if (xmax <= xmin || ymax <= ymin) return false;          // IntersectTile.cu:134
    float ratio = opac / ALPHA_THRESHOLD;
    float k = 0.5f / det_logf(ratio);                        // :156 (reference: __logf)
    conic[0] = conic_in[0] * k; conic[1] = conic_in[1] * k; conic[2] = conic_in[2] * k;
    g.xmin = std::min(std::max(0, f2i(std::floor((xmin + 0.5f) / (float)TILE))), tw);   // :159-162
    g.ymin = std::min(std::max(0, f2i(std::floor((ymin + 0.5f) / (float)TILE))), th);
    g.xmax = std::min(std::max(0, f2i(std::ceil((xmax + 0.5f) / (float)TILE))), tw);
    g.ymax = std::min(std::max(0, f2i(std::ceil((ymax + 0.5f) / (float)TILE))), th);
    return true;
}

// src/core/Common.cuh:55-77
inline bool ellipse_box_overlap_test(float a, float b, float c, float x0, float x1, float y0, float y1) {
    float wx = -b / c, wy = -b / a;
    float u0 = std::min(std::max(x0 * wx, y0), y1);
    float u1 = std::min(std::max(x1 * wx, y0), y1);
    float v0 = std::min(std::max(y0 * wy, x0), x1);
    float v1 = std::min(std::max(y1 * wy, x0), x1);
    b *= 2.0f;
    float mx = std::min(a * x0 * x0 + b * x0 * u0 + c * u0 * u0, a * x1 * x1 + b * x1 * u1 + c * u1 * u1);
    float my = std::min(a * v0 * v0 + b * v0 * y0 + c * y0 * y0, a * v1 * v1 + b * v1 * y1 + c * y1 * y1);
    float mc = std::max(std::max(x0, -x1), std::max(y0, -y1));
    return std::min(mc, std::min(mx, my) - 1.0f) < 0.f;
}

inline bool microtile_hit(const float xy[2], const float conic[3], float opac, int mx, int my) {
    // src/kernels/raster/RasterizationEval3DFwd_kernel.cuh:207-214
    if (!(opac > ALPHA_THRESHOLD)) return false;
    float kk = 0.5f / std::log(opac / ALPHA_THRESHOLD);
    float bx0 = (float)(mx * MICRO), by0 = (float)(my * MICRO);
    return ellipse_box_overlap_test(conic[0] * kk, conic[1] * kk, conic[2] * kk,
                                    bx0 - xy[0], bx0 + MICRO - xy[0], by0 - xy[1], by0 + MICRO - xy[1]);
}

// src/primitives/Primitive3DGS.cuh:250-260 (reference uses __expf)
inline float evaluate_alpha(const float xy[2], const float conic[3], float opac, float px, float py, float* vis_out = nullptr, float* sigma_out = nullptr) {
    float dx = xy[0] - px, dy = xy[1] - py;
    float sigma = 0.5f * (conic[0] * dx * dx + conic[2] * dy * dy) + conic[1] * dx * dy;
    float vis = std::exp(-sigma);
    float alpha = std::min(0.999f, opac * vis);
    if (vis_out) *vis_out = vis;
    if (sigma_out) *sigma_out = sigma;
    return sigma < 0.f ? 0.f : alpha;
}

const float kGauss[11] = {   // src/kernels/loss/FusedSSIM.cu:63-75
    0.001028380123898387f, 0.0075987582094967365f, 0.036000773310661316f, 0.10936068743467331f,
    0.21300552785396576f, 0.26601171493530273f, 0.21300552785396576f, 0.10936068743467331f,
    0.036000773310661316f, 0.0075987582094967365f, 0.001028380123898387f};

}  // namespace

extern "C" {

int oracle_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

float oracle_det_logf(float x) { return det_logf(x); }

// ---------------------------------------------------------------------------
// Projection forward.  projection_3dgs_forward ->
// projection_fused_fwd_kernel (src/kernels/projection/ProjectionFwd_kernel.cuh:15-111)
// Outputs are the reference's arrays: aabb [C*N][4], depths [C*N] (sorting
// depth), radii [N] (max over views; caller zeroes), and the ScreenBuffer
// arrays xy [C*N][2], depth [C*N], conic [C*N][3], opac [C*N], rgb [C*N][3].
// Entries of culled pairs keep aabb = 0 and depths = 0; their screen entries
// are written as zeros here (the reference leaves them untouched).
// ---------------------------------------------------------------------------
void oracle_project_fwd_dist(
    int64_t N, int C, int W, int H, int model, int dist, const float* dist_coeffs, int sh_degree, int antialiased,
    const float* means, const float* quats, const float* scales, const float* opacities,
    const float* features_dc, const float* features_sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_bounds_stride,
    const float* viewmats, const float* intrins,
    float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    ShStore st{features_sh, sh_packed, sh_bounds, sh_bits, sh_bounds_stride > 0 ? sh_bounds_stride : (int64_t)256 * 3 * NUM_SH};
    for (int cid = 0; cid < C; ++cid) {
        Camera cam = load_camera(viewmats, intrins, cid, W, H, model, dist, dist_coeffs);
        if (sh_degree >= 0 && sh_degree <= 3) cam.n_sh = (sh_degree + 1) * (sh_degree + 1) - 1;
#pragma omp parallel for schedule(static)
        for (int64_t gid = 0; gid < N; ++gid) {
            int64_t idx = (int64_t)cid * N + gid;
            float mean[3] = {means[3 * gid], means[3 * gid + 1], means[3 * gid + 2]};
            float quat[4] = {quats[4 * gid], quats[4 * gid + 1], quats[4 * gid + 2], quats[4 * gid + 3]};
            float scale[3] = {scales[3 * gid], scales[3 * gid + 1], scales[3 * gid + 2]};
            float op = opacities[gid];
            ProjResult<float> r;
            projection_3dgs<float>(cam, antialiased != 0, false, mean, quat, scale, op, mean, scale, op, r);
            float col[3] = {0.f, 0.f, 0.f};
            if (r.aabb[2] > r.aabb[0] && r.aabb[3] > r.aabb[1]) {   // src/primitives/Primitive3DGS.cuh:73
                float dc[3] = {features_dc[3 * gid], features_dc[3 * gid + 1], features_dc[3 * gid + 2]};
                float sh[NUM_SH][3];
                for (int j = 0; j < NUM_SH; ++j) for (int ch = 0; ch < 3; ++ch) sh[j][ch] = sh_load(st, gid, j, ch);
                float raw[3], basis[NUM_SH];
                sh_to_color<float>(cam, mean, dc, sh, raw, basis);
                for (int ch = 0; ch < 3; ++ch) col[ch] = std::max(raw[ch] + 0.5f, 0.0f);
            }
            // ProjectionFwd_kernel.cuh:98-110
            float a0 = std::min(std::max(r.aabb[0], 0.0f), (float)W - 1.0f);
            float a1 = std::min(std::max(r.aabb[1], 0.0f), (float)H - 1.0f);
            float a2 = std::min(std::max(r.aabb[2], 0.0f), (float)W - 1.0f);
            float a3 = std::min(std::max(r.aabb[3], 0.0f), (float)H - 1.0f);
            bool keep = (a2 - a0 > 1e-3f) && (a3 - a1 > 1e-3f);
            if (keep) {
                aabb[4 * idx] = a0; aabb[4 * idx + 1] = a1; aabb[4 * idx + 2] = a2; aabb[4 * idx + 3] = a3;
                depths[idx] = r.sorting_depth;
                xy[2 * idx] = r.mean2d[0]; xy[2 * idx + 1] = r.mean2d[1];
                depth[idx] = r.depth;
                conic[3 * idx] = r.conic[0]; conic[3 * idx + 1] = r.conic[1]; conic[3 * idx + 2] = r.conic[2];
                opac[idx] = r.opacity;
                rgb[3 * idx] = col[0]; rgb[3 * idx + 1] = col[1]; rgb[3 * idx + 2] = col[2];
                if (radii) {
                    // atomicMax over views; views are visited one after another here
                    if (r.radius > radii[gid]) radii[gid] = r.radius;
                }
            } else {
                aabb[4 * idx] = aabb[4 * idx + 1] = aabb[4 * idx + 2] = aabb[4 * idx + 3] = 0.f;
                depths[idx] = 0.f;
                xy[2 * idx] = xy[2 * idx + 1] = 0.f; depth[idx] = 0.f;
                conic[3 * idx] = conic[3 * idx + 1] = conic[3 * idx + 2] = 0.f;
                opac[idx] = 0.f; rgb[3 * idx] = rgb[3 * idx + 1] = rgb[3 * idx + 2] = 0.f;
            }
        }
    }
}

void oracle_project_fwd(
    int64_t N, int C, int W, int H, int model, int antialiased,
    const float* means, const float* quats, const float* scales, const float* opacities,
    const float* features_dc, const float* features_sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_bounds_stride,
    const float* viewmats, const float* intrins,
    float* aabb, float* depths, float* radii,
    float* xy, float* depth, float* conic, float* opac, float* rgb) {
    oracle_project_fwd_dist(N, C, W, H, model, 0, nullptr, 3, antialiased, means, quats, scales, opacities, features_dc, features_sh, sh_packed,
                            sh_bounds, sh_bits, sh_bounds_stride, viewmats, intrins, aabb, depths, radii, xy, depth, conic, opac, rgb);
}

// ---------------------------------------------------------------------------
// Projection backward.  projection_3dgs_backward -> projection_fused_bwd_kernel
// (src/kernels/projection/ProjectionBwd_kernel.cuh:16-130): for every pair whose
// stored aabb is non-empty, the vjp of projection_3dgs with assume_valid
// (src/shaders/primitive_3dgs.slang:676-698) plus the SH vjp with the colour
// clamp mask rgb_raw >= -0.5 (src/shaders/harmonics.slang:1087-1126), summed
// into the world gradients (the caller zeroes or pre-loads them).
// ---------------------------------------------------------------------------
void oracle_project_bwd_dist(
    int64_t N, int C, int W, int H, int model, int dist, const float* dist_coeffs, int sh_degree, int antialiased,
    const float* means, const float* quats, const float* scales, const float* opacities,
    const float* features_dc, const float* features_sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_bounds_stride,
    const float* viewmats, const float* intrins, const float* aabb,
    const float* v_xy, const float* v_depth, const float* v_conic, const float* v_opac, const float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    ShStore st{features_sh, sh_packed, sh_bounds, sh_bits, sh_bounds_stride > 0 ? sh_bounds_stride : (int64_t)256 * 3 * NUM_SH};
    constexpr int K = 11;
    typedef Dual<K> D;
    for (int cid = 0; cid < C; ++cid) {
        Camera cam = load_camera(viewmats, intrins, cid, W, H, model, dist, dist_coeffs);
        if (sh_degree >= 0 && sh_degree <= 3) cam.n_sh = (sh_degree + 1) * (sh_degree + 1) - 1;
#pragma omp parallel for schedule(static)
        for (int64_t gid = 0; gid < N; ++gid) {
            int64_t idx = (int64_t)cid * N + gid;
            if (aabb[4 * idx + 2] <= aabb[4 * idx] || aabb[4 * idx + 3] <= aabb[4 * idx + 1]) continue;
            float mean_f[3] = {means[3 * gid], means[3 * gid + 1], means[3 * gid + 2]};
            float scale_f[3] = {scales[3 * gid], scales[3 * gid + 1], scales[3 * gid + 2]};
            D mean[3], quat[4], scale[3], op;
            for (int i = 0; i < 3; ++i) { mean[i] = D(mean_f[i]); mean[i].d[i] = 1.f; }
            for (int i = 0; i < 4; ++i) { quat[i] = D(quats[4 * gid + i]); quat[i].d[3 + i] = 1.f; }
            for (int i = 0; i < 3; ++i) { scale[i] = D(scale_f[i]); scale[i].d[7 + i] = 1.f; }
            op = D(opacities[gid]); op.d[10] = 1.f;
            ProjResult<D> r;
            projection_3dgs<D>(cam, antialiased != 0, true, mean, quat, scale, op, mean_f, scale_f, opacities[gid], r);
            float g[K];
            for (int k = 0; k < K; ++k) {
                g[k] = r.mean2d[0].d[k] * v_xy[2 * idx] + r.mean2d[1].d[k] * v_xy[2 * idx + 1] +
                       r.depth.d[k] * v_depth[idx] +
                       r.conic[0].d[k] * v_conic[3 * idx] + r.conic[1].d[k] * v_conic[3 * idx + 1] + r.conic[2].d[k] * v_conic[3 * idx + 2] +
                       r.opacity.d[k] * v_opac[idx];
            }
            // SH part
            float dc[3] = {features_dc[3 * gid], features_dc[3 * gid + 1], features_dc[3 * gid + 2]};
            float sh[NUM_SH][3];
            for (int j = 0; j < NUM_SH; ++j) for (int ch = 0; ch < 3; ++ch) sh[j][ch] = sh_load(st, gid, j, ch);
            D raw[3], basis[NUM_SH];
            sh_to_color<D>(cam, mean, dc, sh, raw, basis);
            float vc[3];
            for (int ch = 0; ch < 3; ++ch) vc[ch] = v_rgb[3 * idx + ch] * (raw[ch].v >= -0.5f ? 1.f : 0.f);
            for (int k = 0; k < 3; ++k) g[k] += raw[0].d[k] * vc[0] + raw[1].d[k] * vc[1] + raw[2].d[k] * vc[2];
            auto add = [](float* p, float v) { if (std::isfinite(v)) *p += v; };
            for (int i = 0; i < 3; ++i) add(&g_means[3 * gid + i], g[i]);
            for (int i = 0; i < 4; ++i) add(&g_quats[4 * gid + i], g[3 + i]);
            for (int i = 0; i < 3; ++i) add(&g_scales[3 * gid + i], g[7 + i]);
            add(&g_opacities[gid], g[10]);
            for (int ch = 0; ch < 3; ++ch) add(&g_dc[3 * gid + ch], 0.2820947917738781f * vc[ch]);
            for (int j = 0; j < NUM_SH; ++j) for (int ch = 0; ch < 3; ++ch)
                add(&g_sh[(int64_t)3 * NUM_SH * gid + 3 * j + ch], basis[j].v * vc[ch]);
        }
    }
}

void oracle_project_bwd(
    int64_t N, int C, int W, int H, int model, int antialiased,
    const float* means, const float* quats, const float* scales, const float* opacities,
    const float* features_dc, const float* features_sh,
    const uint8_t* sh_packed, const float* sh_bounds, int sh_bits, int64_t sh_bounds_stride,
    const float* viewmats, const float* intrins, const float* aabb,
    const float* v_xy, const float* v_depth, const float* v_conic, const float* v_opac, const float* v_rgb,
    float* g_means, float* g_quats, float* g_scales, float* g_opacities, float* g_dc, float* g_sh) {
    oracle_project_bwd_dist(N, C, W, H, model, 0, nullptr, 3, antialiased, means, quats, scales, opacities, features_dc, features_sh, sh_packed,
                            sh_bounds, sh_bits, sh_bounds_stride, viewmats, intrins, aabb, v_xy, v_depth, v_conic, v_opac, v_rgb,
                            g_means, g_quats, g_scales, g_opacities, g_dc, g_sh);
}

// ---------------------------------------------------------------------------
// Tile intersection: do_intersect_tile_generic, ellipse mode, no live-tile map
// (src/kernels/tile/IntersectTile.cu:372-509).
// Pass 1 (:104-186): tiles_per_splat (int64) and its inclusive sum.
// ---------------------------------------------------------------------------
// tile_active (may be NULL) [I][tile_h][tile_w]: a tile with 0 is left out of both passes, so the rasteriser gets an
// empty range for it (:120-122,164-182,229-258).
int64_t oracle_tile_count_live(
    int64_t total, int64_t N, int W, int H,
    const float* aabb, const float* xy, const float* conic, const float* opac, const int32_t* tile_active,
    int64_t* tiles_per_splat, int64_t* cum_tiles) {
    int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
    for (int64_t idx = 0; idx < total; ++idx) {
        TileSpan g; float cn[3];
        int64_t n = 0;
        const int32_t* live = tile_active ? tile_active + (idx / N) * (int64_t)tw * th : nullptr;
        if (tile_setup(aabb + 4 * idx, conic + 3 * idx, opac[idx], tw, th, g, cn))
            for_each_tile(xy + 2 * idx, cn[0], cn[1], cn[2], g, [&](int x, int y) { if (!live || live[(int64_t)y * tw + x]) ++n; });
        tiles_per_splat[idx] = n;
    }
    int64_t run = 0;
    for (int64_t idx = 0; idx < total; ++idx) { run += tiles_per_splat[idx]; cum_tiles[idx] = run; }
    return run;
}

int64_t oracle_tile_count(
    int64_t total, int W, int H,
    const float* aabb, const float* xy, const float* conic, const float* opac,
    int64_t* tiles_per_splat, int64_t* cum_tiles) {
    return oracle_tile_count_live(total, total > 0 ? total : 1, W, H, aabb, xy, conic, opac, nullptr, tiles_per_splat, cum_tiles);
}

// Pass 2 (:188-267): keys (tile_id << 32 | depth bits) and flatten ids.
void oracle_tile_emit_live(
    int64_t total, int64_t N, int W, int H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac, const int32_t* tile_active,
    const int64_t* cum_tiles, int64_t* isect_ids, int32_t* flatten_ids) {
    int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
#pragma omp parallel for schedule(static)
    for (int64_t idx = 0; idx < total; ++idx) {
        int64_t cur = idx == 0 ? 0 : cum_tiles[idx - 1];
        int64_t end = cum_tiles[idx];
        int64_t iid = idx / N;
        const int32_t* live = tile_active ? tile_active + iid * (int64_t)tw * th : nullptr;
        TileSpan g; float cn[3];
        if (tile_setup(aabb + 4 * idx, conic + 3 * idx, opac[idx], tw, th, g, cn)) {
            float d = std::fabs(depths[idx]);
            uint32_t du; std::memcpy(&du, &d, 4);
            if (du >> 31) du = ~du; else du ^= (1u << 31);       // :190-196
            for_each_tile(xy + 2 * idx, cn[0], cn[1], cn[2], g, [&](int x, int y) {
                if (cur >= end) return;
                if (live && !live[(int64_t)y * tw + x]) return;
                int64_t tile_id = iid * tw * th + (int64_t)y * tw + x;
                isect_ids[cur] = (tile_id << 32) | (int64_t)du;
                flatten_ids[cur] = (int32_t)idx;
                ++cur;
            });
        }
        while (cur < end) {                                      // :261-266
            int64_t tile_id = iid * tw * th;
            isect_ids[cur] = (tile_id << 32) | (int64_t)0xffffffff;
            flatten_ids[cur] = (int32_t)idx;
            ++cur;
        }
    }
}

void oracle_tile_emit(
    int64_t total, int64_t N, int W, int H,
    const float* aabb, const float* depths, const float* xy, const float* conic, const float* opac,
    const int64_t* cum_tiles, int64_t* isect_ids, int32_t* flatten_ids) {
    oracle_tile_emit_live(total, N, W, H, aabb, depths, xy, conic, opac, nullptr, cum_tiles, isect_ids, flatten_ids);
}

// Live-tile map (tile_active_kernel, src/kernels/tile/IntersectTile.cu:309-344): a tile is live when any pixel of it,
// grown by one pixel on every side (kMaskPad) and clipped to the image, is unmasked; the mask [I][Hm][Wm] is sampled
// as the loss samples it (nearest_sample_b, src/core/Interpolation.cuh:108-120).
void oracle_tile_active(const uint8_t* mask, int I, int Hm, int Wm, int W, int H, int32_t* tile_active) {
    const int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
    for (int b = 0; b < I; ++b)
        for (int ty = 0; ty < th; ++ty)
            for (int tx = 0; tx < tw; ++tx) {
                bool live = false;
                for (int dy = -1; dy < TILE + 1 && !live; ++dy) {
                    const int y = ty * TILE + dy;
                    if (y >= H) break;
                    if (y < 0) continue;
                    for (int dx = -1; dx < TILE + 1; ++dx) {
                        const int x = tx * TILE + dx;
                        if (x >= W) break;
                        if (x < 0) continue;
                        float u = ((float)x + 0.5f) * (float)Wm / (float)W - 0.5f;
                        float v = ((float)y + 0.5f) * (float)Hm / (float)H - 0.5f;
                        int xs = std::max(0, std::min(Wm - 1, (int)std::floor(u + 0.5f)));
                        int ys = std::max(0, std::min(Hm - 1, (int)std::floor(v + 0.5f)));
                        if (mask[((size_t)b * Hm + ys) * Wm + xs]) { live = true; break; }
                    }
                }
                tile_active[((size_t)b * th + ty) * tw + tx] = live ? 1 : 0;
            }
}

// Stable ascending sort of (int64 key, int32 value) on key bits
// [begin_bit, end_bit): the contract of cub::DeviceRadixSort::SortPairs as used
// at src/kernels/tile/IntersectTile.cu:487-493 and stated with a CPU oracle in
// src/backend/vulkan/tests/vk_sortscan_test.cpp.
void oracle_sort_pairs(int64_t n, int begin_bit, int end_bit, const int64_t* keys_in, const int32_t* vals_in, int64_t* keys_out, int32_t* vals_out) {
    std::vector<int64_t> order(n);
    std::iota(order.begin(), order.end(), (int64_t)0);
    uint64_t mask = (end_bit - begin_bit >= 64) ? ~0ull : (((1ull << (end_bit - begin_bit)) - 1ull) << begin_bit);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
        return ((uint64_t)keys_in[a] & mask) < ((uint64_t)keys_in[b] & mask);
    });
    for (int64_t i = 0; i < n; ++i) { keys_out[i] = keys_in[order[i]]; vals_out[i] = vals_in[order[i]]; }
}

int oracle_tile_n_bits(int n_tiles) {   // IntersectTile.cu:489-490
    int b = 0;
    while ((1u << b) <= (uint32_t)n_tiles) ++b;
    return b;
}

// intersect_offset_kernel, src/kernels/tile/IntersectTile.cu:271-307; zero when
// there are no intersections (:448-451).
void oracle_tile_offsets(int64_t n_isects, const int64_t* sorted_ids, int64_t n_tiles_total, int32_t* offsets) {
    if (n_isects == 0) { for (int64_t i = 0; i < n_tiles_total; ++i) offsets[i] = 0; return; }
    for (int64_t idx = 0; idx < n_isects; ++idx) {
        int64_t tile_id = sorted_ids[idx] >> 32;
        if (idx == 0) for (int64_t i = 0; i < tile_id + 1; ++i) offsets[i] = (int32_t)idx;
        if (idx == n_isects - 1) for (int64_t i = tile_id + 1; i < n_tiles_total; ++i) offsets[i] = (int32_t)n_isects;
        if (idx > 0) {
            int64_t prev = sorted_ids[idx - 1] >> 32;
            if (prev != tile_id) for (int64_t i = prev + 1; i < tile_id + 1; ++i) offsets[i] = (int32_t)idx;
        }
    }
}

// ---------------------------------------------------------------------------
// Rasterize forward: rasterize_to_pixels_fwd_kernel
// (src/kernels/raster/RasterizationEval3DFwd_kernel.cuh:48-313, 2D variant).
// ---------------------------------------------------------------------------
void oracle_raster_fwd(
    int I, int64_t N, int W, int H, int64_t n_isects,
    const float* xy, const float* depth, const float* conic, const float* opac, const float* rgb,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* out_rgb, float* out_depth, float* out_T, int32_t* last_ids) {
    (void)N;
    int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
    int mw = tw * 2, mh = th * 2;
#pragma omp parallel for schedule(dynamic, 8) collapse(2)
    for (int img = 0; img < I; ++img)
        for (int mt = 0; mt < mw * mh; ++mt) {
            int mt_y = mt / mw, mt_x = mt % mw;
            int tile_id = (mt_y / 2) * tw + (mt_x / 2);
            const int32_t* offs = tile_offsets + (int64_t)img * tw * th;
            int32_t range_start = offs[tile_id];
            int32_t range_end = (img == I - 1 && tile_id == tw * th - 1) ? (int32_t)n_isects : offs[tile_id + 1];
            // per micro-tile hit flags (:207-217)
            std::vector<uint8_t> hit(std::max(0, range_end - range_start));
            for (int32_t k = range_start; k < range_end; ++k) {
                int32_t g = flatten_ids[k];
                hit[k - range_start] = microtile_hit(xy + 2 * g, conic + 3 * g, opac[g], mt_x, mt_y);
            }
            for (int p = 0; p < MICRO * MICRO; ++p) {
                int i = mt_y * MICRO + p / MICRO, j = mt_x * MICRO + p % MICRO;
                if (i >= H || j >= W) continue;
                float px = (float)j + 0.5f, py = (float)i + 0.5f;
                float T = 1.0f; uint32_t cur_idx = 0;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int32_t k = range_start; k < range_end; ++k) {
                    if (!hit[k - range_start]) continue;
                    int32_t g = flatten_ids[k];
                    float alpha = evaluate_alpha(xy + 2 * g, conic + 3 * g, opac[g], px, py);
                    if (alpha <= ALPHA_THRESHOLD) continue;
                    float next_T = T * (1.0f - alpha);
                    if (next_T > 1e-4f) {
                        float vis = alpha * T;
                        acc[0] += rgb[3 * g] * vis; acc[1] += rgb[3 * g + 1] * vis; acc[2] += rgb[3 * g + 2] * vis;
                        acc[3] += depth[g] * vis;
                        cur_idx = (uint32_t)k;
                        T = next_T;
                    } else break;
                }
                int64_t pix = ((int64_t)img * H + i) * W + j;
                out_T[pix] = T;
                float invW = 1.0f / std::max(1.0f - T, 1e-10f);
                out_rgb[3 * pix] = acc[0]; out_rgb[3 * pix + 1] = acc[1]; out_rgb[3 * pix + 2] = acc[2];
                out_depth[pix] = acc[3] * invW;
                last_ids[pix] = (int32_t)cur_idx;
            }
        }
}

// Per-splat densification weight of the raster backward pass (accum_weight_map_buffer -> o_accum_weight,
// src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:541-550,566-579): over every fragment the backward walk
// visits (same skips as oracle_raster_bwd), w = alpha * T0; mode 1: max of map[pixel] * w, mode 2: their sum,
// mode 3: the sum and, in accum_den, the sum of w.  The per-micro-tile partial results the kernel combines with
// atomicMax / atomicAdd are a max / sum over all fragments.  splat = flatten id % N.  Sums in double.
void oracle_raster_accum_weight(
    int I, int64_t N, int W, int H, int64_t n_isects, int mode,
    const float* xy, const float* conic, const float* opac,
    const int32_t* tile_offsets, const int32_t* flatten_ids, const float* render_T, const int32_t* last_ids,
    const float* weight_map, float* accum, float* accum_den) {
    int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
    std::vector<double> acc((size_t)N, 0.0), den((size_t)N, 0.0);
    for (int img = 0; img < I; ++img)
        for (int i = 0; i < H; ++i)
            for (int j = 0; j < W; ++j) {
                int tile_id = (i / TILE) * tw + j / TILE;
                int mt_y = i / MICRO, mt_x = j / MICRO;
                const int32_t* offs = tile_offsets + (int64_t)img * tw * th;
                int32_t range_start = offs[tile_id];
                int32_t range_end = (img == I - 1 && tile_id == tw * th - 1) ? (int32_t)n_isects : offs[tile_id + 1];
                int64_t pix = ((int64_t)img * H + i) * W + j;
                float px = (float)j + 0.5f, py = (float)i + 0.5f;
                float T1 = render_T[pix];
                float wm = weight_map ? weight_map[pix] : 0.f;
                for (int32_t k = std::min(range_end - 1, last_ids[pix]); k >= range_start; --k) {
                    int32_t g = flatten_ids[k];
                    if (!microtile_hit(xy + 2 * g, conic + 3 * g, opac[g], mt_x, mt_y)) continue;
                    float vis, sigma;
                    float alpha = evaluate_alpha(xy + 2 * g, conic + 3 * g, opac[g], px, py, &vis, &sigma);
                    if (alpha <= ALPHA_THRESHOLD) continue;
                    float T0 = T1 * (1.0f / (1.0f - alpha));
                    float w = alpha * T0;
                    int64_t wid = (int64_t)g % N;
                    if (mode == 1) acc[wid] = std::max(acc[wid], (double)(wm * w));
                    else acc[wid] += (double)wm * (double)w;
                    den[wid] += (double)w;
                    T1 = T0;
                }
            }
    for (int64_t n = 0; n < N; ++n) {
        accum[n] = (float)acc[n];
        if (mode == 3 && accum_den) accum_den[n] = (float)den[n];
    }
}

// ---------------------------------------------------------------------------
// Rasterize backward: rasterize_to_pixels_bwd_kernel
// (src/kernels/raster/RasterizationEval3DBwd_kernel.cuh:48-636, 2D variant) with
// the fragment vjp of src/primitives/Primitive3DGS.cuh:262-300.  Per-splat sums
// are formed in double and rounded once (the reference adds floats atomically
// in a run-dependent order).  Gradients are ADDED to the v_* arrays.
// ---------------------------------------------------------------------------
void oracle_raster_bwd(
    int I, int64_t N, int W, int H, int64_t n_isects,
    const float* xy, const float* depth, const float* conic, const float* opac, const float* rgb,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    const float* render_depth, const float* render_T, const int32_t* last_ids,
    const float* v_render_rgb, const float* v_render_depth, const float* v_render_T,
    float* v_xy, float* v_depth, float* v_conic, float* v_opac, float* v_rgb) {
    (void)N;
    int tw = (W + TILE - 1) / TILE, th = (H + TILE - 1) / TILE;
    int mw = tw * 2, mh = th * 2;
    // one 10-vector per (pair, micro-tile slot): pair k, slot = which of the 4 micro-tiles
    std::vector<double> pg((size_t)n_isects * 10, 0.0);
    // micro-tiles of one macro tile share pair rows -> process a whole macro tile per task
#pragma omp parallel for schedule(dynamic, 4) collapse(2)
    for (int img = 0; img < I; ++img)
        for (int tile_id = 0; tile_id < tw * th; ++tile_id) {
            const int32_t* offs = tile_offsets + (int64_t)img * tw * th;
            int32_t range_start = offs[tile_id];
            int32_t range_end = (img == I - 1 && tile_id == tw * th - 1) ? (int32_t)n_isects : offs[tile_id + 1];
            int ty = tile_id / tw, tx = tile_id % tw;
            for (int sub = 0; sub < 4; ++sub) {
                int mt_y = ty * 2 + sub / 2, mt_x = tx * 2 + sub % 2;
                if (mt_y >= mh || mt_x >= mw) continue;
                for (int p = 0; p < MICRO * MICRO; ++p) {
                    int i = mt_y * MICRO + p / MICRO, j = mt_x * MICRO + p % MICRO;
                    if (i >= H || j >= W) continue;
                    int64_t pix = ((int64_t)img * H + i) * W + j;
                    float px = (float)j + 0.5f, py = (float)i + 0.5f;
                    int32_t bin_final = last_ids[pix];
                    float T1 = render_T[pix];
                    float v_T1 = v_render_T ? v_render_T[pix] : 0.f;
                    float vc[4] = {v_render_rgb[3 * pix], v_render_rgb[3 * pix + 1], v_render_rgb[3 * pix + 2], v_render_depth ? v_render_depth[pix] : 0.f};
                    {   // :214-228
                        float inv_alpha = 1.0f / std::max(1.0f - T1, 1e-10f);
                        float exp_depth = render_depth[pix];
                        v_T1 += exp_depth * vc[3] * inv_alpha;
                        vc[3] *= inv_alpha;
                    }
                    for (int32_t k = std::min(range_end - 1, bin_final); k >= range_start; --k) {
                        int32_t g = flatten_ids[k];
                        if (!microtile_hit(xy + 2 * g, conic + 3 * g, opac[g], mt_x, mt_y)) continue;
                        float vis, sigma;
                        float alpha = evaluate_alpha(xy + 2 * g, conic + 3 * g, opac[g], px, py, &vis, &sigma);
                        if (alpha <= ALPHA_THRESHOLD) continue;
                        float ra = 1.0f / (1.0f - alpha);
                        float T0 = T1 * ra;
                        float cdot = rgb[3 * g] * vc[0] + rgb[3 * g + 1] * vc[1] + rgb[3 * g + 2] * vc[2] + depth[g] * vc[3];
                        float v_alpha = T0 * cdot - v_T1 * T0;                  // :482
                        float w = alpha * T0;
                        float v_T0 = alpha * cdot + v_T1 * (1.0f - alpha);      // :494
                        double* o = &pg[(size_t)k * 10];
                        // evaluate_alpha_vjp, Primitive3DGS.cuh:262-286
                        if (sigma >= 0.f && opac[g] * vis <= 0.999f) {
                            float dx = xy[2 * g] - px, dy = xy[2 * g + 1] - py;
                            float v_sigma = -opac[g] * vis * v_alpha;
                            o[3] += 0.5f * v_sigma * dx * dx;
                            o[4] += v_sigma * dx * dy;
                            o[5] += 0.5f * v_sigma * dy * dy;
                            o[0] += v_sigma * (conic[3 * g] * dx + conic[3 * g + 1] * dy);
                            o[1] += v_sigma * (conic[3 * g + 1] * dx + conic[3 * g + 2] * dy);
                            o[6] += vis * v_alpha;
                        }
                        o[7] += vc[0] * w; o[8] += vc[1] * w; o[9] += vc[2] * w;  // :488, evaluate_color_vjp
                        o[2] += vc[3] * w;
                        T1 = T0; v_T1 = v_T0;
                    }
                }
            }
        }
    // fold pair rows into splat rows
    std::vector<double> sg;
    int64_t max_g = 0;
    for (int64_t k = 0; k < n_isects; ++k) max_g = std::max<int64_t>(max_g, flatten_ids[k]);
    sg.assign((size_t)(max_g + 1) * 10, 0.0);
    for (int64_t k = 0; k < n_isects; ++k) {
        int32_t g = flatten_ids[k];
        for (int c = 0; c < 10; ++c) sg[(size_t)g * 10 + c] += pg[(size_t)k * 10 + c];
    }
    for (int64_t g = 0; g <= max_g && n_isects > 0; ++g) {
        const double* s = &sg[(size_t)g * 10];
        v_xy[2 * g] += (float)s[0]; v_xy[2 * g + 1] += (float)s[1];
        v_depth[g] += (float)s[2];
        v_conic[3 * g] += (float)s[3]; v_conic[3 * g + 1] += (float)s[4]; v_conic[3 * g + 2] += (float)s[5];
        v_opac[g] += (float)s[6];
        v_rgb[3 * g] += (float)s[7]; v_rgb[3 * g + 1] += (float)s[8]; v_rgb[3 * g + 2] += (float)s[9];
    }
}

// ---------------------------------------------------------------------------
// Loss: w_l1 * mean|render-gt| + w_ssim * (1 - SSIM), one scale, no masks.
// Per-pixel part: src/shaders/per_pixel_losses.slang:133-176 (RgbLoss, L1 term)
// reduced by :365-375, whose reverse gives v_rgb = w_l1 * sign(r-g) / (3*B*P).
// SSIM part: memory_efficient_ssim_backward_kernel<inplace>
// (src/kernels/loss/FusedSSIM.cu:639-1022) with dL_dmap = -w_ssim, added in place.
// losses[0] = L1 mean, losses[1] = SSIM mean, losses[2] = total.
// ---------------------------------------------------------------------------
// map_mode (SsimLossMapMode, src/kernels/loss/PerPixelLoss.cuh:129-134) != 0: loss_map[b][y][x] +=
// map_weight * (1 - mean over channels of v), v = SSIM (1), D/B (2), D / (2 sqrt(s1 s2) + C2) (3);
// FusedSSIM.cu:861-886,1009-1016.
//
// mask (may be NULL) [Bm][Hm][Wm] bytes, != 0 = the pixel takes part.  Read as get_pix_value does
// (FusedSSIM.cu:105-126) and nearest_sample_b (src/core/Interpolation.cuh:108-120): nearest sample when its
// size is not the image's, and every tap outside the image (or an image index >= Bm) reads unmasked.
//   per-pixel part (per_pixel_losses.slang:161-176,290-291,365-375): masked pixels add nothing to the L1 sum and
//     get no gradient; the sum is divided by max(number of unmasked pixels of the batch, 1).
//   SSIM part (FusedSSIM.cu:717-724,829-848,858-887,902-915,988-994): masked samples are dropped from the
//     window sums, the sums are divided by the window's coverage (Gaussian weight on unmasked taps,
//     :138-177), a window centred on a masked pixel scores 1 and sends no gradient, a masked pixel
//     receives none, and its loss-map value is that of a perfect match.
// map_l1 != 0 (DensifyLossMapMode::LossFull, PerPixelLoss.cu:1127-1131, :200-217): the pixel's weighted
//   L1 term |mask * w_l1 * mean_c |r - g|| is added to the loss map as well.
static inline bool mask_tap(const uint8_t* mask, int b, int y, int x, int Bm, int Hm, int Wm, int H, int W) {
    if (!mask) return true;
    if ((unsigned)b >= (unsigned)Bm || (unsigned)x >= (unsigned)W || (unsigned)y >= (unsigned)H) return true;
    int xs = x, ys = y;
    if (Wm != W || Hm != H) {
        float u = ((float)x + 0.5f) * (float)Wm / (float)W - 0.5f;
        float v = ((float)y + 0.5f) * (float)Hm / (float)H - 0.5f;
        xs = std::max(0, std::min(Wm - 1, (int)std::floor(u + 0.5f)));
        ys = std::max(0, std::min(Hm - 1, (int)std::floor(v + 0.5f)));
    }
    return mask[((size_t)b * Hm + ys) * Wm + xs] != 0;
}

void oracle_loss_l1_ssim_masked(
    int B, int H, int W, float w_l1, float w_ssim,
    const float* render, const float* gt, const uint8_t* mask, int Bm, int Hm, int Wm,
    float* v_render, float* losses, int map_mode, float map_weight, int map_l1, float* loss_map) {
    const int64_t P = (int64_t)H * W;
    std::vector<float> lm_sum(map_mode ? (size_t)B * P : 0, 0.f);
    std::vector<uint8_t> mk((size_t)B * P, 1);
    double mask_total = (double)B * P;
    if (mask) {
        mask_total = 0.0;
        for (int b = 0; b < B; ++b)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    bool m = mask_tap(mask, b, y, x, Bm, Hm, Wm, H, W);
                    mk[(size_t)b * P + (size_t)y * W + x] = m;
                    mask_total += m;
                }
    }
    double l1_sum = 0.0, ssim_sum = 0.0;
    const float inv_mask_total = 1.0f / std::max((float)mask_total, 1.0f);
#pragma omp parallel for reduction(+ : l1_sum) schedule(static)
    for (int64_t i = 0; i < (int64_t)B * P; ++i) {
        float s = 0.f;
        const float m = mk[i] ? 1.f : 0.f;
        for (int ch = 0; ch < 3; ++ch) {
            float d = render[3 * i + ch] - gt[3 * i + ch];
            s += std::fabs(d);
            float sg = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
            v_render[3 * i + ch] = m * w_l1 * sg * (1.0f / 3.0f) * inv_mask_total;
        }
        l1_sum += (double)(m * s * (1.0f / 3.0f));
        if (map_l1 && loss_map) loss_map[i] += std::fabs(m * w_l1 * (s * (1.0f / 3.0f)));
    }
    const float grad = -w_ssim / (3.0f * B * W * H);   // FusedSSIM.cu:667
    const float kC1 = 0.01f * 0.01f, kC2 = 0.03f * 0.03f;
    for (int b = 0; b < B; ++b) {
        // coverage of every window (FusedSSIM.cu:138-177); rows outside the image count as unmasked
        std::vector<float> cov;
        if (mask) {
            std::vector<float> tmp(P);
            cov.resize(P);
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    float acc = 0.f;
                    for (int d = -5; d <= 5; ++d) acc += kGauss[5 - std::abs(d)] * (float)mask_tap(mask, b, y, x + d, Bm, Hm, Wm, H, W);
                    tmp[(size_t)y * W + x] = acc;
                }
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    float acc = 0.f;
                    for (int d = -5; d <= 5; ++d) {
                        int yy = y + d;
                        float row = (unsigned)yy < (unsigned)H ? tmp[(size_t)yy * W + x] : 0.9999999f;
                        acc += kGauss[5 - std::abs(d)] * row;
                    }
                    cov[(size_t)y * W + x] = acc;
                }
        }
        const uint8_t* mb = mk.data() + (size_t)b * P;
        for (int ch = 0; ch < 3; ++ch) {
            // horizontal pass of the five moments, zero padding; masked samples are dropped
            std::vector<float> hx(P), hx2(P), hy(P), hy2(P), hxy(P);
            auto X = [&](int y, int x) { return render[3 * ((int64_t)b * P + (int64_t)y * W + x) + ch]; };
            auto Y = [&](int y, int x) { return gt[3 * ((int64_t)b * P + (int64_t)y * W + x) + ch]; };
#pragma omp parallel for schedule(static)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    float sx = 0, sx2 = 0, sy = 0, sy2 = 0, sxy = 0;
                    for (int d = -5; d <= 5; ++d) {
                        int xx = x + d;
                        if (xx < 0 || xx >= W || !mb[(size_t)y * W + xx]) continue;
                        float w = kGauss[d + 5], a = X(y, xx), c = Y(y, xx);
                        sx += a * w; sx2 += a * a * w; sy += c * w; sy2 += c * c * w; sxy += a * c * w;
                    }
                    int64_t o = (int64_t)y * W + x;
                    hx[o] = sx; hx2[o] = sx2; hy[o] = sy; hy2[o] = sy2; hxy[o] = sxy;
                }
            std::vector<float> d_mu1(P), d_s1(P), d_s12(P);
            double csum = 0.0;
#pragma omp parallel for reduction(+ : csum) schedule(static)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    float o0 = 0, o1 = 0, o2 = 0, o3 = 0, o4 = 0;
                    for (int d = -5; d <= 5; ++d) {
                        int yy = y + d;
                        if (yy < 0 || yy >= H) continue;
                        float w = kGauss[d + 5];
                        int64_t o = (int64_t)yy * W + x;
                        o0 += hx[o] * w; o1 += hx2[o] * w; o2 += hy[o] * w; o3 += hy2[o] * w; o4 += hxy[o] * w;
                    }
                    int64_t o = (int64_t)y * W + x;
                    const float inv_cov = mask ? 1.0f / std::max(cov[o], 1e-6f) : 1.0f;
                    const bool cmask = mb[o] != 0;
                    // FusedSSIM.cu:822-848,891-915
                    float mu1 = o0 * inv_cov, mu2 = o2 * inv_cov;
                    float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
                    float sigma1_sq = o1 * inv_cov - mu1_sq, sigma2_sq = o3 * inv_cov - mu2_sq, sigma12 = o4 * inv_cov - mu1 * mu2;
                    float A = mu1_sq + mu2_sq + kC1;
                    float Bv = sigma1_sq + sigma2_sq + kC2;
                    float C_ = 2.f * mu1 * mu2 + kC1;
                    float D_ = 2.f * sigma12 + kC2;
                    float ssim_v = (C_ * D_) / (A * Bv);
                    csum += cmask ? (double)ssim_v : 1.0;
                    if (map_mode) {
                        float lm = ssim_v;
                        if (map_mode == 2) lm = D_ / Bv;
                        else if (map_mode == 3) lm = D_ / (2.f * std::sqrt(std::max(sigma1_sq, 0.0f) * std::max(sigma2_sq, 0.0f)) + kC2);
                        if (!cmask) lm = 1.0f;
                        lm_sum[(size_t)b * P + o] += lm;
                    }
                    const float g = cmask ? grad * inv_cov : 0.f;
                    d_mu1[o] = ((mu2 * 2.f * D_) / (A * Bv) - (mu2 * 2.f * C_) / (A * Bv) - (mu1 * 2.f * C_ * D_) / (A * A * Bv) + (mu1 * 2.f * C_ * D_) / (A * Bv * Bv)) * g;
                    d_s1[o] = ((-C_ * D_) / (A * Bv * Bv)) * g;
                    d_s12[o] = ((2.f * C_) / (A * Bv)) * g;
                }
            ssim_sum += csum;
            // second separable convolution of the three partial maps (:903-1000)
            std::vector<float> t0(P), t1(P), t2(P);
#pragma omp parallel for schedule(static)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    float a0 = 0, a1 = 0, a2 = 0;
                    for (int d = -5; d <= 5; ++d) {
                        int xx = x + d;
                        if (xx < 0 || xx >= W) continue;
                        float w = kGauss[d + 5];
                        int64_t o = (int64_t)y * W + xx;
                        a0 += d_mu1[o] * w; a1 += d_s1[o] * w; a2 += d_s12[o] * w;
                    }
                    int64_t o = (int64_t)y * W + x;
                    t0[o] = a0; t1[o] = a1; t2[o] = a2;
                }
#pragma omp parallel for schedule(static)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    if (!mb[(size_t)y * W + x]) continue;   // a masked pixel receives no gradient (:988-994)
                    float s0 = 0, s1 = 0, s2 = 0;
                    for (int d = -5; d <= 5; ++d) {
                        int yy = y + d;
                        if (yy < 0 || yy >= H) continue;
                        float w = kGauss[d + 5];
                        int64_t o = (int64_t)yy * W + x;
                        s0 += t0[o] * w; s1 += t1[o] * w; s2 += t2[o] * w;
                    }
                    float p1 = X(y, x), p2 = Y(y, x);
                    v_render[3 * ((int64_t)b * P + (int64_t)y * W + x) + ch] += s0 + (2.f * p1) * s1 + p2 * s2;   // :990-1000
                }
        }
    }
    float l1 = (float)(l1_sum / std::max(mask_total, 1.0));
    float ssim = (float)(ssim_sum / (double)(3.0 * B * P));
    if (losses) { losses[0] = l1; losses[1] = ssim; losses[2] = w_l1 * l1 + w_ssim * (1.0f - ssim); }
    if (map_mode)
        for (int64_t i = 0; i < (int64_t)B * P; ++i) loss_map[i] += map_weight * (1.0f - lm_sum[i] / 3.0f);
}

void oracle_loss_l1_ssim_map(
    int B, int H, int W, float w_l1, float w_ssim,
    const float* render, const float* gt, float* v_render, float* losses,
    int map_mode, float map_weight, float* loss_map) {
    oracle_loss_l1_ssim_masked(B, H, W, w_l1, w_ssim, render, gt, nullptr, 0, 0, 0, v_render, losses, map_mode, map_weight, 0, loss_map);
}

// ---------------------------------------------------------------------------
// Multi-scale loss: compute_multi_scale_per_pixel_losses (src/kernels/loss/PerPixelLoss.cu:941-1363)
// restricted to the colour modalities (render, target, mask).
//   pyramid (:1032-1097): every level halves the previous one (max(1, n / 2)).  Images pool 2x2; where a mask of the
//     image's own size exists the pool is the mean over the unmasked children, or the plain mean when all four are
//     masked (avg_pool_downsample_masked_float_kernel, :675-701).  The mask pools to "at least two of four"
//     (avg_pool_downsample_bool_kernel, :723-740), halving ITS OWN size.
//   every level (:1106-1232): the per-pixel pass writes the level's gradient, the SSIM pass adds to it; loss-map modes
//     (DensifyLossMapMode, PerPixelLoss.cuh:98-110): 1 = per-pixel term + w_ssim * (1 - SSIM), 2/3/4 = w_ssim * (1 - SSIM / CS / structure).
//   fold (:1262-1325): gradient = (g_0 + sum_s 0.25^s * up(g_s)) / S and loss map = (m_0 + sum_s up(m_s)) / S, with
//     up(a)[y][x] = a[y >> s][x >> s] where that exists and 0 elsewhere (avg_pool_upsample_float_kernel, :926-943);
//     with a mask of the image's size and S > 1 the masked pixels' gradient is cleared at the end (:1327-1336).
//   losses (:1256-1259,1338-1345): mean over the levels; the SSIM value reported is level 0's (:1252-1253).
// losses[0] = mean L1, losses[1] = level-0 SSIM, losses[2] = mean over levels of w_l1 * L1 + w_ssim * (1 - SSIM).
// ---------------------------------------------------------------------------
void oracle_loss_multi_scale(
    int B, int H, int W, int num_scales, float w_l1, float w_ssim,
    const float* render, const float* gt, const uint8_t* mask, int Hm, int Wm,
    float* v_render, float* losses, int loss_map_mode, float* loss_map) {
    struct Level { int H, W, Hm, Wm; std::vector<float> r, g, v, lm; std::vector<uint8_t> m; };
    std::vector<Level> lv(num_scales);
    lv[0].H = H; lv[0].W = W; lv[0].Hm = Hm; lv[0].Wm = Wm;
    lv[0].r.assign(render, render + (size_t)B * H * W * 3);
    lv[0].g.assign(gt, gt + (size_t)B * H * W * 3);
    if (mask) lv[0].m.assign(mask, mask + (size_t)B * Hm * Wm);
    for (int s = 1; s < num_scales; ++s) {
        const Level& a = lv[s - 1];
        Level& c = lv[s];
        c.H = std::max(1, a.H / 2); c.W = std::max(1, a.W / 2);
        const bool same = mask && a.Hm == a.H && a.Wm == a.W;
        auto at = [&](const std::vector<float>& img, int b, int y, int x, int ch) {   // TensorView::at clamps nothing: 2y+1 < H holds for H >= 2
            y = std::min(y, a.H - 1); x = std::min(x, a.W - 1);
            return img[(((size_t)b * a.H + y) * a.W + x) * 3 + ch];
        };
        auto pool = [&](const std::vector<float>& src, std::vector<float>& dst) {
            dst.resize((size_t)B * c.H * c.W * 3);
            for (int b = 0; b < B; ++b)
                for (int y = 0; y < c.H; ++y)
                    for (int x = 0; x < c.W; ++x)
                        for (int ch = 0; ch < 3; ++ch) {
                            float acc = 0.f, box = 0.f;
                            int n = 0;
                            for (int dy = 0; dy < 2; ++dy)
                                for (int dx = 0; dx < 2; ++dx) {
                                    float v = at(src, b, 2 * y + dy, 2 * x + dx, ch);
                                    bool valid = same ? a.m[((size_t)b * a.H + std::min(2 * y + dy, a.H - 1)) * a.W + std::min(2 * x + dx, a.W - 1)] != 0 : false;
                                    box += 0.25f * v;
                                    if (valid) { acc += v; ++n; }
                                }
                            float out;
                            if (same) out = n ? acc / (float)n : box;
                            else out = 0.25f * (at(src, b, 2 * y, 2 * x, ch) + at(src, b, 2 * y, 2 * x + 1, ch) + at(src, b, 2 * y + 1, 2 * x, ch) +
                                                at(src, b, 2 * y + 1, 2 * x + 1, ch));
                            dst[(((size_t)b * c.H + y) * c.W + x) * 3 + ch] = out;
                        }
        };
        pool(a.r, c.r);
        pool(a.g, c.g);
        c.Hm = c.Wm = 0;
        if (mask) {
            c.Hm = std::max(1, a.Hm / 2); c.Wm = std::max(1, a.Wm / 2);
            c.m.resize((size_t)B * c.Hm * c.Wm);
            for (int b = 0; b < B; ++b)
                for (int y = 0; y < c.Hm; ++y)
                    for (int x = 0; x < c.Wm; ++x) {
                        int v = 0;
                        for (int dy = 0; dy < 2; ++dy)
                            for (int dx = 0; dx < 2; ++dx)
                                v += a.m[((size_t)b * a.Hm + std::min(2 * y + dy, a.Hm - 1)) * a.Wm + std::min(2 * x + dx, a.Wm - 1)] != 0;
                        c.m[((size_t)b * c.Hm + y) * c.Wm + x] = v >= 2;
                    }
        }
    }
    const int ssim_mode = loss_map_mode == 1 || loss_map_mode == 2 ? 1 : (loss_map_mode == 3 ? 2 : (loss_map_mode == 4 ? 3 : 0));
    double l1_mean = 0.0, tot_mean = 0.0;
    float ssim0 = 0.f;
    for (int s = 0; s < num_scales; ++s) {
        Level& c = lv[s];
        c.v.assign((size_t)B * c.H * c.W * 3, 0.f);
        if (loss_map) c.lm.assign((size_t)B * c.H * c.W, 0.f);
        float l[3];
        oracle_loss_l1_ssim_masked(B, c.H, c.W, w_l1, w_ssim, c.r.data(), c.g.data(), mask ? c.m.data() : nullptr, B, c.Hm, c.Wm, c.v.data(), l,
                                   loss_map ? ssim_mode : 0, w_ssim, loss_map && loss_map_mode == 1, loss_map ? c.lm.data() : nullptr);
        l1_mean += l[0] / num_scales;
        tot_mean += l[2] / num_scales;
        if (s == 0) ssim0 = l[1];
    }
    const float inv_s = 1.0f / (float)num_scales;
    for (int b = 0; b < B; ++b)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x) {
                const size_t p = ((size_t)b * H + y) * W + x;
                float g[3] = {lv[0].v[3 * p], lv[0].v[3 * p + 1], lv[0].v[3 * p + 2]};
                float m = loss_map ? lv[0].lm[p] : 0.f;
                for (int s = 1; s < num_scales; ++s) {
                    const Level& c = lv[s];
                    const int ys = y >> s, xs = x >> s;
                    if (ys >= c.H || xs >= c.W) continue;
                    const size_t q = ((size_t)b * c.H + ys) * c.W + xs;
                    const float wgt = std::pow(0.25f, (float)s);
                    for (int ch = 0; ch < 3; ++ch) g[ch] += wgt * c.v[3 * q + ch];
                    if (loss_map) m += c.lm[q];
                }
                const bool keep = !(num_scales > 1 && mask && Hm == H && Wm == W && !mask[p]);
                for (int ch = 0; ch < 3; ++ch) v_render[3 * p + ch] = num_scales > 1 ? (keep ? g[ch] * inv_s : 0.f) : g[ch];
                if (loss_map) loss_map[p] = num_scales > 1 ? m * inv_s : m;
            }
    if (losses) { losses[0] = (float)l1_mean; losses[1] = ssim0; losses[2] = (float)tot_mean; }
}

void oracle_loss_l1_ssim(
    int B, int H, int W, float w_l1, float w_ssim,
    const float* render, const float* gt, float* v_render, float* losses) {
    oracle_loss_l1_ssim_map(B, H, W, w_l1, w_ssim, render, gt, v_render, losses, 0, 0.f, nullptr);
}

// ---------------------------------------------------------------------------
// Adam, geometry attributes: fused_optim_3dgs_geometry_kernel
// (src/kernels/optim/FusedGeometryOptim.cu:83-380) with every per-splat
// regulariser weight zero, no scale-agnostic mean, fp32 state, scalar step.
// ---------------------------------------------------------------------------
void oracle_adam_geometry_ex(
    int64_t N, int step, float grad_scale, int zero_grad,
    float lr_means, float lr_quats, float lr_scales, float lr_opacs,
    float* means, float* v_means, float* g1_means, float* g2_means,
    float* quats, float* v_quats, float* g1_quats, float* g2_quats,
    float* scales, float* v_scales, float* g1_scales, float* g2_scales,
    float* opacs, float* v_opacs, float* g1_opacs, float* g2_opacs,
    // regulariser weights as the caller gives them (the launcher divides them by N, :457-462), in the order
    // max_gauss_ratio, scale_regularization, mcmc_opacity, mcmc_scale, erank, erank_s3, quat_norm
    const float* reg, int use_scale_agnostic_mean, const float* radii, const int32_t* steps, float* densify_score) {
    const float eps = 1e-15f, beta1 = 0.9f, beta2 = 0.999f;
    const float lr_means0 = lr_means, lr_quats0 = lr_quats, lr_scales0 = lr_scales, lr_opacs0 = lr_opacs;
    const float inv_n = 1.0f / (float)N;
    const float max_ratio = reg ? reg[0] : 0.f, w_ratio = reg ? reg[1] * inv_n : 0.f, w_op = reg ? reg[2] * inv_n : 0.f,
                w_ms = reg ? reg[3] * inv_n : 0.f, w_er = reg ? reg[4] * inv_n : 0.f, w_er3 = reg ? reg[5] * inv_n : 0.f,
                w_qn = reg ? reg[6] * inv_n : 0.f;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < N; ++i) {
        const float stepf = (float)(steps ? steps[i] : step);   // :160
        const float ibc1 = 1.0f / (1.0f - std::pow(beta1, stepf));
        const float ibc2 = 1.0f / (1.0f - std::pow(beta2, stepf));
        const float lr_means = lr_means0 * ibc1, lr_quats = lr_quats0 * ibc1, lr_scales = lr_scales0 * ibc1, lr_opacs = lr_opacs0 * ibc1;
        auto upd = [&](float& x, float g, float& m1, float& m2, float lr) {
            m1 = beta1 * m1 + (1.f - beta1) * g;
            m2 = beta2 * m2 + (1.f - beta2) * g * g;
            x = x - lr * m1 / (std::sqrt(m2 * ibc2) + eps);
        };
        // parameters before the update (:170-172), used by the regularisers and the scale-agnostic mean
        const float s0[3] = {scales[3 * i], scales[3 * i + 1], scales[3 * i + 2]};
        const float o0 = opacs[i];
        float qn0[4];
        {
            float n = 0.f;
            for (int k = 0; k < 4; ++k) n += quats[4 * i + k] * quats[4 * i + k];
            float inv = 1.0f / std::sqrt(n);
            for (int k = 0; k < 4; ++k) qn0[k] = quats[4 * i + k] * inv;
        }
        // reverse mode of per_splat_losses with unit cotangents (src/shaders/per_splat_losses.slang:5-141)
        float rs[3] = {0.f, 0.f, 0.f}, ro = 0.f, rq[4] = {0.f, 0.f, 0.f, 0.f};
        if (reg) {
            const float sg = 1.0f / (1.0f + std::exp(-o0));
            ro = w_op * sg * (1.0f - sg);                                             // mcmc_opacity_reg, :61-65
            for (int k = 0; k < 3; ++k) rs[k] = w_ms * 1e-2f / 3.0f;                  // mcmc_scale_reg_3dgs, :69-73
            int imax = s0[0] > s0[1] ? 0 : 1; imax = s0[imax] > s0[2] ? imax : 2;
            int imin = s0[0] < s0[1] ? 0 : 1; imin = s0[imin] < s0[2] ? imin : 2;
            const float ratio = std::exp(s0[imax]) / std::exp(s0[imin]);              // scale_reg_3dgs, :41-46
            if (ratio > max_ratio) { rs[imax] += w_ratio * ratio; rs[imin] -= w_ratio * ratio; }
            {                                                                          // erank_reg_3dgs, :9-20
                const float E[3] = {std::exp(2.0f * s0[0]), std::exp(2.0f * s0[1]), std::exp(2.0f * s0[2])};
                const float S = E[0] + E[1] + E[2];
                const float p1 = E[imax] / S, p3 = E[imin] / S, p2 = 1.0f - p1 - p3;
                const float l1 = std::log(p1), l2 = std::log(p2), l3 = std::log(p3);
                const float r = std::exp(-p1 * l1 - p2 * l2 - p3 * l3);
                float dH = 0.f;
                if (-std::log(r - 0.99999f) > 0.0f) dH = -w_er / (r - 0.99999f) * r;
                const float dp1 = dH * (l2 - l1), dp3 = dH * (l2 - l3) + w_er3;
                const float dS = -(dp1 * p1 + dp3 * p3) / S;
                for (int k = 0; k < 3; ++k) {
                    float dE = dS + (k == imax ? dp1 / S : 0.f) + (k == imin ? dp3 / S : 0.f);
                    rs[k] += dE * 2.0f * E[k];
                }
            }
            {                                                                          // quat_norm_reg, :84-88
                float n = std::sqrt(qn0[0] * qn0[0] + qn0[1] * qn0[1] + qn0[2] * qn0[2] + qn0[3] * qn0[3]);
                float w = w_qn * (1.0f - 1.0f / n) / n;
                for (int k = 0; k < 4; ++k) rq[k] = w * qn0[k];
            }
        }
        for (int k = 0; k < 3; ++k) {
            float g = rs[k] + grad_scale * v_scales[3 * i + k];
            upd(scales[3 * i + k], g, g1_scales[3 * i + k], g2_scales[3 * i + k], lr_scales);
            if (zero_grad) v_scales[3 * i + k] = 0.f;
        }
        {   // Riemannian quaternion step, :231-243
            float q[4], g[4];
            float n = 0.f;
            for (int k = 0; k < 4; ++k) { q[k] = quats[4 * i + k]; n += q[k] * q[k]; }
            float inv = 1.0f / std::sqrt(n);
            for (int k = 0; k < 4; ++k) q[k] *= inv;
            float dotqg = 0.f;
            for (int k = 0; k < 4; ++k) { g[k] = rq[k] + grad_scale * v_quats[4 * i + k]; dotqg += q[k] * g[k]; }
            for (int k = 0; k < 4; ++k) g[k] -= dotqg * q[k];
            float u[4]; float n2 = 0.f;
            for (int k = 0; k < 4; ++k) {
                float& m1 = g1_quats[4 * i + k]; float& m2 = g2_quats[4 * i + k];
                m1 = beta1 * m1 + (1.f - beta1) * g[k];
                m2 = beta2 * m2 + (1.f - beta2) * g[k] * g[k];
                u[k] = q[k] - lr_quats * m1 / (std::sqrt(m2 * ibc2) + eps);
                n2 += u[k] * u[k];
            }
            float inv2 = 1.0f / std::sqrt(n2);
            for (int k = 0; k < 4; ++k) { quats[4 * i + k] = u[k] * inv2; if (zero_grad) v_quats[4 * i + k] = 0.f; }
        }
        {
            float g = ro + grad_scale * v_opacs[i];
            upd(opacs[i], g, g1_opacs[i], g2_opacs[i], lr_opacs);
            if (zero_grad) v_opacs[i] = 0.f;
        }
        if (densify_score) {   // :283-286, from the gradient and the log-scales before the update
            const float vx = grad_scale * v_means[3 * i], vy = grad_scale * v_means[3 * i + 1], vz = grad_scale * v_means[3 * i + 2];
            densify_score[i] = std::exp(std::max(std::max(s0[0], s0[1]), s0[2])) * std::sqrt(vx * vx + vy * vy + vz * vz);
        }
        if (use_scale_agnostic_mean) {   // :302-314
            const float v[3] = {grad_scale * v_means[3 * i], grad_scale * v_means[3 * i + 1], grad_scale * v_means[3 * i + 2]};
            const float w = qn0[0], x = qn0[1], y = qn0[2], z = qn0[3];
            const float R[9] = {1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y),
                                2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x),
                                2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)};
            // apply_covar_to_vec(quat, exp(s/2), v) = R diag(exp(s)) R^T v (src/shaders/projection_utils.slang:114-161)
            float t[3];
            for (int k = 0; k < 3; ++k) t[k] = std::exp(s0[k]) * (R[k] * v[0] + R[3 + k] * v[1] + R[6 + k] * v[2]);
            const float sg = 1.0f / (1.0f + std::exp(-o0));
            const float ext = std::sqrt(2.0f * std::log(std::max(255.0f * sg, 1.00001f)));
            const float den = radii[i] * 0.6f;
            for (int k = 0; k < 3; ++k) {
                const float num = (R[3 * k] * t[0] + R[3 * k + 1] * t[1] + R[3 * k + 2] * t[2]) * ext;
                float& m1 = g1_means[3 * i + k]; float& m2 = g2_means[3 * i + k];
                m1 = beta1 * m1 + (1.f - beta1) * num;
                m2 = beta2 * m2 + (1.f - beta2) * v[k] * v[k] * den * den;
                means[3 * i + k] -= lr_means * m1 / (std::sqrt(m2 * ibc2) + eps);
                if (zero_grad) v_means[3 * i + k] = 0.f;
            }
        } else {
            for (int k = 0; k < 3; ++k) {
                float g = grad_scale * v_means[3 * i + k];
                upd(means[3 * i + k], g, g1_means[3 * i + k], g2_means[3 * i + k], lr_means);
                if (zero_grad) v_means[3 * i + k] = 0.f;
            }
        }
    }
}

void oracle_adam_geometry(
    int64_t N, int step, float grad_scale, int zero_grad,
    float lr_means, float lr_quats, float lr_scales, float lr_opacs,
    float* means, float* v_means, float* g1_means, float* g2_means,
    float* quats, float* v_quats, float* g1_quats, float* g2_quats,
    float* scales, float* v_scales, float* g1_scales, float* g2_scales,
    float* opacs, float* v_opacs, float* g1_opacs, float* g2_opacs) {
    oracle_adam_geometry_ex(N, step, grad_scale, zero_grad, lr_means, lr_quats, lr_scales, lr_opacs, means, v_means, g1_means, g2_means,
                            quats, v_quats, g1_quats, g2_quats, scales, v_scales, g1_scales, g2_scales, opacs, v_opacs, g1_opacs, g2_opacs,
                            nullptr, 0, nullptr, nullptr, nullptr);
}

// fused_adam_step -> fused_adam_with_steps_kernel
// (src/kernels/optim/FusedAppearanceOptim.cu:11-92); decay = 2*l2_reg/numel.
void oracle_adam_plain_steps(
    int64_t numel, int step, float lr, float l2_reg, float l2_reg_offset, float grad_scale, int zero_grad,
    float* param, float* grad, float* exp_avg, float* exp_avg_sq, const int32_t* steps, int stride) {
    const float eps = 1e-15f, beta1 = 0.9f, beta2 = 0.999f;
    const float decay = 2.0f * l2_reg / (float)numel;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < numel; ++i) {
        const float stepf = (float)(steps ? steps[i / stride] : step);   // :34
        const float ibc1 = 1.0f / (1.0f - std::pow(beta1, stepf));
        const float ibc2 = 1.0f / (1.0f - std::pow(beta2, stepf));
        float x = param[i], v = grad[i];
        if (!std::isfinite(v)) v = 0.f;
        if (zero_grad) grad[i] = 0.f;
        v *= grad_scale;
        v += decay * (std::max(x - l2_reg_offset, 0.0f) + std::min(x + l2_reg_offset, 0.0f));
        float g1 = beta1 * exp_avg[i] + (1.f - beta1) * v;
        float g2 = beta2 * exp_avg_sq[i] + (1.f - beta2) * v * v;
        x -= lr * ibc1 * g1 / (std::sqrt(g2 * ibc2) + eps);
        param[i] = x; exp_avg[i] = g1; exp_avg_sq[i] = g2;
    }
}

void oracle_adam_plain(
    int64_t numel, int step, float lr, float l2_reg, float l2_reg_offset, float grad_scale, int zero_grad,
    float* param, float* grad, float* exp_avg, float* exp_avg_sq) {
    oracle_adam_plain_steps(numel, step, lr, l2_reg, l2_reg_offset, grad_scale, zero_grad, param, grad, exp_avg, exp_avg_sq, nullptr, 1);
}

// Block-wise min/max value codec, QuantizedTensor<BITS,256>::encode_v
// (src/core/Tensor.h:1380-1393): bounds[b] = (min, max) of block b of 256 cells.
void oracle_quant_encode(int64_t numel, int bits, const float* values, uint8_t* packed, float* bounds) {
    const float qmax = (float)((1 << bits) - 1);
    int64_t nb = (numel + 255) / 256;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        int64_t lo = b * 256, hi = std::min(numel, lo + 256);
        float mn = 1e30f, mx = -1e30f;
        for (int64_t i = lo; i < hi; ++i) { mn = std::min(mn, values[i]); mx = std::max(mx, values[i]); }
        bounds[2 * b] = mn; bounds[2 * b + 1] = mx;
        float range = std::max(mx - mn, 1e-30f);
        for (int64_t i = lo; i < hi; ++i) {
            float qf = std::round(qmax * (values[i] - mn) / range);
            qf = std::min(std::max(qf, 0.0f), qmax);
            if (bits == 8) packed[i] = (uint8_t)qf;
            else reinterpret_cast<uint16_t*>(packed)[i] = (uint16_t)qf;
        }
    }
}

void oracle_quant_decode(int64_t numel, int bits, const uint8_t* packed, const float* bounds, float* values) {
    const float inv = 1.0f / (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < numel; ++i) {
        const float* mm = bounds + 2 * (i / 256);
        float q = bits == 8 ? (float)packed[i] : (float)reinterpret_cast<const uint16_t*>(packed)[i];
        values[i] = mm[0] + (mm[1] - mm[0]) * (q * inv);
    }
}

// Doubly-quantised Adam for SH: fused_adam_with_steps_qq_kernel<256, 8, VALUE_BITS>
// (src/kernels/optim/FusedAppearanceOptim.cu:291-418) with the state codec
// QuantizedAdamState<8,256> (src/core/Tensor.h:978-1136) and the value codec
// QuantizedTensor<VALUE_BITS,256> (:1313-1404).  fp32 gradient input.
// value_bits == 32: the values are plain fp32 and only the state is quantised
// (fused_adam_with_steps_8bit_kernel, src/kernels/optim/FusedAppearanceOptim.cu:137-229).
void oracle_adam_qq_ex(
    int64_t numel, int step, float lr, float l2_reg, float l2_reg_offset, float grad_scale, int zero_grad, int value_bits,
    float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed, float* value_bounds,
    const int32_t* steps, int stride, int optim_bits) {
    const float eps = 1e-15f, beta1 = 0.9f, beta2 = 0.999f, kEps = 1e-15f;
    const float decay = 2.0f * l2_reg / (float)numel;
    const bool plain = value_bits == 32;
    const float vq = plain ? 1.0f : (float)((1 << value_bits) - 1), vinv = 1.0f / vq;
    // QuantizedAdamState<4|8,256>: 4 bits = one byte per cell, u in the low nibble (src/core/Tensor.h:1051-1054)
    const bool nib = optim_bits == 4;
    const float oq = nib ? 15.0f : 255.0f, oinv = 1.0f / oq;
    int64_t nb = (numel + 255) / 256;
    float* value_f32 = reinterpret_cast<float*>(value_packed);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        int64_t lo = b * 256, hi = std::min(numel, lo + 256);
        float xs[256], us[256], ss[256];
        float vmm[2] = {plain ? 0.f : value_bounds[2 * b], plain ? 0.f : value_bounds[2 * b + 1]};
        float omm[4] = {optim_bounds[4 * b], optim_bounds[4 * b + 1], optim_bounds[4 * b + 2], optim_bounds[4 * b + 3]};
        float nv[2] = {1e30f, -1e30f}, no[4] = {1e30f, -1e30f, 1e30f, -1e30f};
        for (int64_t i = lo; i < hi; ++i) {
            float q = plain ? 0.f : value_bits == 8 ? (float)value_packed[i] : (float)reinterpret_cast<uint16_t*>(value_packed)[i];
            float x = plain ? value_f32[i] : vmm[0] + (vmm[1] - vmm[0]) * (q * vinv);
            float v = grad[i];
            if (!std::isfinite(v)) v = 0.f;
            if (zero_grad) grad[i] = 0.f;
            v *= grad_scale;
            v += decay * (std::max(x - l2_reg_offset, 0.0f) + std::min(x + l2_reg_offset, 0.0f));
            float u_q = nib ? (float)(optim_packed[i] & 15) : (float)optim_packed[2 * i];
            float s_q = nib ? (float)(optim_packed[i] >> 4) : (float)optim_packed[2 * i + 1];
            float u = omm[0] + (omm[1] - omm[0]) * (u_q * oinv);
            float ls = omm[2] + (omm[3] - omm[2]) * (s_q * oinv);
            float sqrt_g2 = kEps * std::expm1(ls);
            float g1 = u * (sqrt_g2 + kEps), g2 = sqrt_g2 * sqrt_g2;
            g1 = beta1 * g1 + (1.f - beta1) * v;
            g2 = beta2 * g2 + (1.f - beta2) * v * v;
            const float stepf = (float)(steps ? steps[i / stride] : step);   // :166, :330
            const float ibc1 = 1.0f / (1.0f - std::pow(beta1, stepf));
            const float ibc2 = 1.0f / (1.0f - std::pow(beta2, stepf));
            x -= lr * ibc1 * g1 / (std::sqrt(g2 * ibc2) + eps);
            float sq = std::sqrt(std::max(g2, 0.0f));
            float un = g1 / (sq + kEps);
            float sn = std::log1p(std::max(sq, 0.0f) * (1.0f / kEps));
            xs[i - lo] = x; us[i - lo] = un; ss[i - lo] = sn;
            nv[0] = std::min(nv[0], x); nv[1] = std::max(nv[1], x);
            no[0] = std::min(no[0], un); no[1] = std::max(no[1], un);
            no[2] = std::min(no[2], sn); no[3] = std::max(no[3], sn);
        }
        float vrange = std::max(nv[1] - nv[0], 1e-30f);
        float urange = std::max(no[1] - no[0], kEps), srange = std::max(no[3] - no[2], kEps);
        for (int64_t i = lo; i < hi; ++i) {
            float qf = std::min(std::max(std::round(vq * (xs[i - lo] - nv[0]) / vrange), 0.0f), vq);
            if (plain) value_f32[i] = xs[i - lo];
            else if (value_bits == 8) value_packed[i] = (uint8_t)qf;
            else reinterpret_cast<uint16_t*>(value_packed)[i] = (uint16_t)qf;
            float uq = std::min(std::max(std::round(oq * (us[i - lo] - no[0]) / urange), 0.0f), oq);
            float sq = std::min(std::max(std::round(oq * (ss[i - lo] - no[2]) / srange), 0.0f), oq);
            if (nib) optim_packed[i] = (uint8_t)((uint8_t)uq | ((uint8_t)sq << 4));
            else { optim_packed[2 * i] = (uint8_t)uq; optim_packed[2 * i + 1] = (uint8_t)sq; }
        }
        if (!plain) { value_bounds[2 * b] = nv[0]; value_bounds[2 * b + 1] = nv[1]; }
        for (int k = 0; k < 4; ++k) optim_bounds[4 * b + k] = no[k];
    }
}

// The SH section of the reference's fused backward + optimiser at quantisation level 1
// (fused_projection_bwd_optimizer_3dgs_kernel<..., 256, 8, VALUE_BITS>, src/kernels/optim/FusedProjectionBwdOptim_kernel.cuh:709-975):
// the same two codecs, with one float4 of state bounds and one float2 of value bounds per 256 SPLATS (all 45 cells of each).
// n_active = live cells per splat (3 * coefficients of the active degree); the idle cells are not updated but written as zero
// value / zero moments against bounds widened to contain zero (:836-857, :918-925).  Regulariser: 2 l2 / (45 n) * value (:769-773
// with the wrapper's scaling :1137 and the division by num_sh :695).
void oracle_adam_sh_splat_blocks(
    int64_t n_splats, int n_active, int step, float lr, float l2_reg, float grad_scale, int value_bits,
    const float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed, float* value_bounds, const int32_t* steps) {
    const float eps = 1e-15f, beta1 = 0.9f, beta2 = 0.999f, kEps = 1e-15f;
    if (n_active <= 0) return;
    const float decay = 2.0f * l2_reg / (float)(n_splats * 45);
    const float vq = (float)((1 << value_bits) - 1), vinv = 1.0f / vq, oq = 255.0f, oinv = 1.0f / 255.0f;
    const int64_t nb = (n_splats + 255) / 256;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t lo = b * 256 * 45, hi = std::min(n_splats, (b + 1) * 256) * 45;
        std::vector<float> xs(hi - lo, 0.f), us(hi - lo, 0.f), ss(hi - lo, 0.f);
        const float vmm[2] = {value_bounds[2 * b], value_bounds[2 * b + 1]};
        const float omm[4] = {optim_bounds[4 * b], optim_bounds[4 * b + 1], optim_bounds[4 * b + 2], optim_bounds[4 * b + 3]};
        float nv[2] = {1e30f, -1e30f}, no[4] = {1e30f, -1e30f, 1e30f, -1e30f};
        for (int64_t i = lo; i < hi; ++i) {
            if (i % 45 >= n_active) continue;
            const float q = value_bits == 8 ? (float)value_packed[i] : (float)reinterpret_cast<uint16_t*>(value_packed)[i];
            float x = vmm[0] + (vmm[1] - vmm[0]) * (q * vinv);
            float v = grad[i];
            if (!std::isfinite(v)) v = 0.f;
            v *= grad_scale;
            v += decay * x;
            const float u = omm[0] + (omm[1] - omm[0]) * ((float)optim_packed[2 * i] * oinv);
            const float ls = omm[2] + (omm[3] - omm[2]) * ((float)optim_packed[2 * i + 1] * oinv);
            const float sqrt_g2 = kEps * std::expm1(ls);
            float g1 = u * (sqrt_g2 + kEps), g2 = sqrt_g2 * sqrt_g2;
            g1 = beta1 * g1 + (1.f - beta1) * v;
            g2 = beta2 * g2 + (1.f - beta2) * v * v;
            const float stepf = (float)(steps ? steps[i / 45] : step);
            const float ibc1 = 1.0f / (1.0f - std::pow(beta1, stepf)), ibc2 = 1.0f / (1.0f - std::pow(beta2, stepf));
            x -= lr * ibc1 * g1 / (std::sqrt(g2 * ibc2) + eps);
            const float sq = std::sqrt(std::max(g2, 0.0f));
            const float un = g1 / (sq + kEps), sn = std::log1p(sq * (1.0f / kEps));
            xs[i - lo] = x; us[i - lo] = un; ss[i - lo] = sn;
            nv[0] = std::min(nv[0], x); nv[1] = std::max(nv[1], x);
            no[0] = std::min(no[0], un); no[1] = std::max(no[1], un);
            no[2] = std::min(no[2], sn); no[3] = std::max(no[3], sn);
        }
        if (n_active < 45) {
            nv[0] = std::min(nv[0], 0.f); nv[1] = std::max(nv[1], 0.f);
            no[0] = std::min(no[0], 0.f); no[1] = std::max(no[1], 0.f); no[2] = std::min(no[2], 0.f);
        }
        const float vrange = std::max(nv[1] - nv[0], 1e-30f), urange = std::max(no[1] - no[0], kEps), srange = std::max(no[3] - no[2], kEps);
        for (int64_t i = lo; i < hi; ++i) {
            const float qf = std::min(std::max(std::round(vq * (xs[i - lo] - nv[0]) / vrange), 0.0f), vq);
            if (value_bits == 8) value_packed[i] = (uint8_t)qf; else reinterpret_cast<uint16_t*>(value_packed)[i] = (uint16_t)qf;
            optim_packed[2 * i] = (uint8_t)std::min(std::max(std::round(oq * (us[i - lo] - no[0]) / urange), 0.0f), oq);
            optim_packed[2 * i + 1] = (uint8_t)std::min(std::max(std::round(oq * (ss[i - lo] - no[2]) / srange), 0.0f), oq);
        }
        value_bounds[2 * b] = nv[0]; value_bounds[2 * b + 1] = nv[1];
        for (int k = 0; k < 4; ++k) optim_bounds[4 * b + k] = no[k];
    }
}

void oracle_adam_qq(
    int64_t numel, int step, float lr, float l2_reg, float l2_reg_offset, float grad_scale, int zero_grad, int value_bits,
    float* grad, uint8_t* optim_packed, float* optim_bounds, uint8_t* value_packed, float* value_bounds) {
    oracle_adam_qq_ex(numel, step, lr, l2_reg, l2_reg_offset, grad_scale, zero_grad, value_bits, grad, optim_packed, optim_bounds,
                      value_packed, value_bounds, nullptr, 1, 8);
}


// ---------------------------------------------------------------------------
// Densification, per-step part (src/engine/EngineDensify.cpp:193-263,355-367).
// ---------------------------------------------------------------------------

// Quantile of the strictly positive finite entries of x[0], x[stride], ... with every copy of the maximum left out, by the
// lower-rank convention rank = (uint)(clamp(q) * (count - 1)) evaluated in float; 1 when there is no such entry and
// max / 2 when all of them are the maximum (select_pass_kernel, src/kernels/densify/Quantile.cu:164-243).  Stated here by
// sorting, as a check of the radix select.
float oracle_quantile_positive(const float* x, int64_t n, int64_t stride, float q) {
    std::vector<float> v;
    float mx = 0.f;
    for (int64_t i = 0; i < n; ++i) {
        float a = x[i * stride];
        if (a > 0.f && std::isfinite(a)) { v.push_back(a); mx = std::max(mx, a); }
    }
    if (v.empty()) return 1.0f;
    std::vector<float> w;
    for (float a : v) if (a != mx) w.push_back(a);
    if (w.empty()) return mx * 0.5f;
    std::sort(w.begin(), w.end());
    uint32_t rank = (uint32_t)(std::min(1.0f, std::max(0.0f, q)) * (float)(w.size() - 1));
    return w[rank];
}

static inline float hash14_ref(float a, float b, float c, float d) {   // DensifyScoring.cu:200-206
    a = std::fmod(a * .1031f, 1.0f); b = std::fmod(b * .1030f, 1.0f); c = std::fmod(c * .0973f, 1.0f); d = std::fmod(d * .1099f, 1.0f);
    const float dt = a * (d + 33.33f) + b * (c + 33.33f) + c * (a + 33.33f) + d * (b + 33.33f);
    a += dt; b += dt; c += dt; d += dt;
    return std::fmod((a + b) * (c + d), 1.0f);
}

// densify_clip_scale_kernel (DensifyScoring.cu:150-178) + densify_accum_finalize_kernel (:281-291) +
// densify_update_weight_kernel (:213-276) + densify_clip_score_kernel (:319-343), buffers chosen as
// engine_densify_step chooses them (EngineDensify.cpp:211-263).  accum_mode 3 = averaged raster weights.
void oracle_densify_update_scores(
    int64_t n, float max_scale2d, float clip_hardness, float max_scale3d, int accum_mode, int score_mode, float blend_w, float score_power,
    float clip_quantile, float final_power, const float* radii, float* log_scales, const float* logit_opacs, float* accum_weight,
    const float* accum_den, const float* world_grad, float* accum_buffer, float* sample_score) {
    for (int64_t i = 0; i < n; ++i) {
        if (std::isfinite(max_scale2d)) {
            float over = radii[i] / max_scale2d;
            if (std::isfinite(clip_hardness)) over = std::min(over, clip_hardness);
            if (over > 1.0f) {
                float l = std::log(over);
                for (int k = 0; k < 3; ++k) log_scales[3 * i + k] -= l;
            }
        }
        if (std::isfinite(max_scale3d)) {
            float cap = std::log(max_scale3d);
            for (int k = 0; k < 3; ++k) log_scales[3 * i + k] = std::min(log_scales[3 * i + k], cap);
        }
    }
    if (!accum_buffer) return;
    if (accum_mode == 3 && accum_weight)
        for (int64_t i = 0; i < n; ++i) accum_weight[i] = accum_den[i] > 0.f ? accum_weight[i] / accum_den[i] : 0.f;
    const float* score = accum_weight;
    const float* score2 = nullptr;
    bool by_opacity = false;
    if (blend_w >= 1.0f && world_grad) score = world_grad;
    else if (accum_weight) { if (blend_w > 0.0f && world_grad) score2 = world_grad; }
    else { score = logit_opacs; by_opacity = true; }
    for (int64_t i = 0; i < n; ++i) {
        if (!(radii[i] > 0.f)) continue;
        float weight = std::fabs(score[i]);
        if (score2) {
            weight = std::pow(weight, 1.0f - blend_w) * std::pow(std::fabs(score2[i]), blend_w);
            if (!std::isfinite(weight)) weight = 0.f;
        }
        if (by_opacity) weight *= 1.0f / (1.0f + std::exp(-logit_opacs[i]));
        if (weight == 0.f) continue;
        if (score_power != 1.0f) weight = std::pow(weight, score_power);
        float ax = accum_buffer[2 * i], ay = accum_buffer[2 * i + 1];
        if (score_mode == 1) { ax = std::max(ax, weight); ay = std::max(ay, 1.0f); }
        else if (score_mode == 0) { ax = (ax * ay + weight) / (ay + 1.0f); ay += 1.0f; }
        else if (score_mode == 2) {
            float r = hash14_ref(1e2f * weight, 1e2f * ax, 1e2f * ay, 1e2f * (ay + 1.5f));
            if (ay == 0.f) { ax = weight * std::exp2(r - 0.5f); ay = 1.0f; }
            else { ax *= std::exp2((weight > ax ? 1.0f : -1.0f) * r); ay += 1.0f; }
        } else {
            ax = std::exp((std::log(std::max(ax, 1e-30f)) * ay + std::log(std::max(weight, 1e-30f))) / (ay + 1.0f));
            ay += 1.0f;
        }
        accum_buffer[2 * i] = ax; accum_buffer[2 * i + 1] = ay;
    }
    const bool clip = clip_quantile > 0.f && clip_quantile < 1.f;
    if (!clip && !sample_score) return;
    const float c = clip ? oracle_quantile_positive(accum_buffer, n, 2, clip_quantile) : 0.f;
    for (int64_t i = 0; i < n; ++i) {
        float v = accum_buffer[2 * i];
        if (clip && c > 0.f && !(v <= c)) { v = c; accum_buffer[2 * i] = c; }
        if (sample_score) {
            if (final_power != 1.0f) v = std::pow(std::max(v, 0.0f), final_power);
            sample_score[2 * i] = v; sample_score[2 * i + 1] = accum_buffer[2 * i + 1];
        }
    }
}

// mcmc_add_noise_3dgs / revised_add_noise_3dgs (src/shaders/densify.slang:13-74): three unit normals from hash44 + Box-Muller
// of the splat's own parameters (src/shaders/projection_utils.slang:37-68), shaped by R diag(s^2) R^T (MCMC) or R diag(s) R^T
// (revised).  z_out (optional, [n][3]) receives the normals, so a caller can check the shaping apart from the hash.
void oracle_densify_add_noise(int64_t n, float scaler, int revised, const float* radii, float* means, const float* log_scales,
                              const float* quats, const float* logit_opacs, float* z_out) {
    auto fract = [](float x) { return x - std::floor(x); };
    for (int64_t i = 0; i < n; ++i) {
        if (revised && radii[i] <= 0.f) continue;
        const float* m = means + 3 * i; const float* l = log_scales + 3 * i; const float* q = quats + 4 * i;
        const float opac = 1.0f / (1.0f + std::exp(-logit_opacs[i]));
        float a = m[0] * m[0] + m[1] * m[1] + m[2] * m[2], b = m[0] * l[0] + m[1] * l[1] + m[2] * l[2], c = l[0] * l[0] + l[1] * l[1] + l[2] * l[2],
              d = (q[0] + q[1] + q[2] + q[3]) * opac;
        a = fract(a * .1031f); b = fract(b * .1030f); c = fract(c * .0973f); d = fract(d * .1099f);
        const float dt = a * (d + 33.33f) + b * (c + 33.33f) + c * (a + 33.33f) + d * (b + 33.33f);
        a += dt; b += dt; c += dt; d += dt;
        const float hx = fract((a + b) * c), hy = fract((a + c) * b), hz = fract((b + c) * d), hw = fract((c + d) * a);
        const float r0 = std::sqrt(-2.0f * std::log(1.0f - hx)), r1 = std::sqrt(-2.0f * std::log(1.0f - hy));
        const float z[3] = {r0 * std::cos(6.28318530718f * hz), r0 * std::sin(6.28318530718f * hz), r1 * std::cos(6.28318530718f * hw)};
        if (z_out) { z_out[3 * i] = z[0]; z_out[3 * i + 1] = z[1]; z_out[3 * i + 2] = z[2]; }
        const float inv = 1.0f / std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
        const float w = q[0] * inv, x = q[1] * inv, y = q[2] * inv, zq = q[3] * inv;
        const float R[3][3] = {{1.f - 2.f * (y * y + zq * zq), 2.f * (x * y - w * zq), 2.f * (x * zq + w * y)},
                               {2.f * (x * y + w * zq), 1.f - 2.f * (x * x + zq * zq), 2.f * (y * zq - w * x)},
                               {2.f * (x * zq - w * y), 2.f * (y * zq + w * x), 1.f - 2.f * (x * x + y * y)}};
        float s[3], amp;
        if (revised) {
            for (int k = 0; k < 3; ++k) s[k] = std::exp(l[k]);
            amp = std::min(0.05f * scaler * std::sqrt(2.0f * std::log(std::max(255.0f * opac, 1.0f))) * std::pow(1.0f - opac, 150.0f), 1.0f);
        } else {
            for (int k = 0; k < 3; ++k) s[k] = std::exp(2.f * l[k]);
            amp = scaler * (1.0f / (1.0f + std::exp(-100.0f * ((1.0f - opac) - 0.995f))));
        }
        float t[3];
        for (int k = 0; k < 3; ++k) t[k] = s[k] * (R[0][k] * z[0] + R[1][k] * z[1] + R[2][k] * z[2]) * amp;
        for (int r = 0; r < 3; ++r) means[3 * i + r] = m[r] + R[r][0] * t[0] + R[r][1] * t[1] + R[r][2] * t[2];
    }
}


// ---------------------------------------------------------------------------
// Densification, periodic part: relocation of dead splats and growth by the long-axis split
// (relocate_splats_with_long_axis_split_tensor / add_splats_with_long_axis_split_tensor,
// src/kernels/densify/Relocation.cu:205-369).
// ---------------------------------------------------------------------------
static inline uint32_t hash_uint3_ref(uint32_t a, uint32_t b, uint32_t c) {      // src/core/Common.cuh:1019-1039
    uint32_t h = a;
    h *= 0x01000193u; h = (h << 16) | (h >> 16);
    h ^= b; h *= 0x01000193u; h = (h << 16) | (h >> 16);
    h ^= c; h *= 0x01000193u;
    h ^= h >> 15; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}

// Indices of the k smallest Efraimidis-Spirakis keys w / log(1 - u), ties by index (a stable ascending sort, as the
// reference's radix sort of (key, index); DensifySampling.cu:278-390).  weights: [n][2], the score in lane 0.  alive: may be NULL.
void oracle_weighted_sample(int64_t n, uint32_t seed, const float* weights, const uint8_t* alive, int64_t k, int32_t* out) {
    std::vector<float> key(n);
    for (int64_t i = 0; i < n; ++i) {
        float u = (float)hash_uint3_ref(seed, (uint32_t)(i >> 8), (uint32_t)(i & 255)) * 2.3283064365386963e-10f;
        float w = weights[2 * i] / det_logf(std::max(1.0f - u, 1e-30f));
        if (alive && !alive[i]) w = 0.0f;
        if (w == 0.0f) w = 0.0f;
        key[i] = w;
    }
    std::vector<int32_t> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return key[a] < key[b]; });
    for (int64_t i = 0; i < k; ++i) out[i] = order[i];
}

struct OracleDensifyArrays {
    float *means, *quats, *scales, *opacs, *dc, *sh;
    float *m1[6], *m2[6];
    uint8_t* sh_optim_packed; float* sh_optim_bounds; int sh_optim_bits;
    uint8_t* sh_value_packed; float* sh_value_bounds; int sh_value_bits;
    float* accum; int32_t* steps;
};

static void split_one(const OracleDensifyArrays& a, int64_t s, int64_t d, float split_k) {   // Relocation.cu:13-157, densify.slang:76-94
    const float lx = a.scales[3 * s], ly = a.scales[3 * s + 1], lz = a.scales[3 * s + 2];
    const float* q = a.quats + 4 * s;
    const float op = a.opacs[s];
    const float dlen = 0.5f * std::exp(std::max(std::max(lx, ly), lz));
    const float kl = std::log(0.5f), ks = std::log(0.85f);
    float n3[3] = {lx, ly, lz}, e[3] = {0.f, 0.f, 0.f};
    if (lx > ly && lx > lz) { n3[0] += kl; n3[1] += ks; n3[2] += ks; e[0] = dlen; }
    else if (ly > lz) { n3[0] += ks; n3[1] += kl; n3[2] += ks; e[1] = dlen; }
    else { n3[0] += ks; n3[1] += ks; n3[2] += kl; e[2] = dlen; }
    const float inv = 1.0f / std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
    const float w = q[0] * inv, x = q[1] * inv, y = q[2] * inv, z = q[3] * inv;
    const float R[3][3] = {{1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y)},
                           {2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x)},
                           {2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)}};
    const float new_op = std::log(split_k / (1.0f + std::exp(-op) - split_k));
    for (int r = 0; r < 3; ++r) {
        const float dl = R[r][0] * e[0] + R[r][1] * e[1] + R[r][2] * e[2];
        const float m = a.means[3 * s + r];
        a.means[3 * s + r] = m - dl; a.means[3 * d + r] = m + dl;
        a.scales[3 * s + r] = n3[r]; a.scales[3 * d + r] = n3[r];
    }
    a.opacs[s] = new_op; a.opacs[d] = new_op;
    for (int k = 0; k < 4; ++k) a.quats[4 * d + k] = q[k];
    for (int k = 0; k < 3; ++k) a.dc[3 * d + k] = a.dc[3 * s + k];
    if (a.sh) for (int k = 0; k < 45; ++k) a.sh[45 * d + k] = a.sh[45 * s + k];
    if (a.sh_value_bits != 32 && a.sh_value_packed) {                                   // DensifyQuantCopy.cuh:37-77
        const float qmax = a.sh_value_bits == 16 ? 65535.0f : 255.0f;
        for (int k = 0; k < 45; ++k) {
            const int64_t cs = 45 * s + k, cd = 45 * d + k;
            const float* ms = a.sh_value_bounds + 2 * (cs >> 8); const float* md = a.sh_value_bounds + 2 * (cd >> 8);
            const float code = a.sh_value_bits == 16 ? (float)((const uint16_t*)a.sh_value_packed)[cs] : (float)a.sh_value_packed[cs];
            const float v = ms[0] + (ms[1] - ms[0]) * (code * (1.0f / qmax));
            const float qf = std::min(std::max(std::round(qmax * (v - md[0]) / std::max(md[1] - md[0], 1e-30f)), 0.0f), qmax);
            if (a.sh_value_bits == 16) ((uint16_t*)a.sh_value_packed)[cd] = (uint16_t)qf; else a.sh_value_packed[cd] = (uint8_t)qf;
        }
    }
    const int width[6] = {3, 4, 3, 1, 3, 45};
    for (int t = 0; t < 6; ++t)
        if (a.m1[t]) for (int k = 0; k < width[t]; ++k) { a.m1[t][(int64_t)width[t] * d + k] = 0.f; a.m2[t][(int64_t)width[t] * d + k] = 0.f; }
    if (a.sh_optim_bits && a.sh_optim_packed) {                                         // DensifyQuantCopy.cuh:29-35,234-269
        const float qmax = a.sh_optim_bits == 8 ? 255.0f : 15.0f;
        auto zero_code = [&](float lo, float hi) { return (uint32_t)std::min(std::max(std::round(qmax * (0.0f - lo) / std::max(hi - lo, 1e-30f)), 0.0f), qmax); };
        for (int k = 0; k < 45; ++k) {
            const int64_t c = 45 * d + k;
            const float* mm = a.sh_optim_bounds + 4 * (c >> 8);
            const uint32_t uq = zero_code(mm[0], mm[1]), sq = zero_code(mm[2], mm[3]);
            if (a.sh_optim_bits == 8) { a.sh_optim_packed[2 * c] = (uint8_t)uq; a.sh_optim_packed[2 * c + 1] = (uint8_t)sq; }
            else a.sh_optim_packed[c] = (uint8_t)((uq & 15u) | ((sq & 15u) << 4));
        }
    }
    if (a.steps) a.steps[d] = 0;
    if (a.accum) { a.accum[2 * d] = a.accum[2 * s]; a.accum[2 * d + 1] = a.accum[2 * s + 1]; }
}

// mode 0: relocate (dead slots in ascending order; returns their number; src_out / dst_out receive the pairs);
// mode 1: add num_new splats at cur_n...
int64_t oracle_densify_split(
    int mode, int64_t cur_n, int64_t num_new, float min_opacity, float split_k, uint32_t seed, const float* weights,
    float* means, float* quats, float* scales, float* opacs, float* dc, float* sh,
    float* m1_means, float* m1_quats, float* m1_scales, float* m1_opacs, float* m1_dc, float* m1_sh,
    float* m2_means, float* m2_quats, float* m2_scales, float* m2_opacs, float* m2_dc, float* m2_sh,
    uint8_t* sh_optim_packed, float* sh_optim_bounds, int sh_optim_bits, uint8_t* sh_value_packed, float* sh_value_bounds, int sh_value_bits,
    float* accum, int32_t* steps, int32_t* src_out, int32_t* dst_out) {
    OracleDensifyArrays a{means, quats, scales, opacs, dc, sh, {m1_means, m1_quats, m1_scales, m1_opacs, m1_dc, m1_sh},
                          {m2_means, m2_quats, m2_scales, m2_opacs, m2_dc, m2_sh}, sh_optim_packed, sh_optim_bounds, sh_optim_bits,
                          sh_value_packed, sh_value_bounds, sh_value_bits, accum, steps};
    std::vector<uint8_t> alive;
    std::vector<int32_t> dst;
    int64_t count = num_new;
    if (mode == 0) {
        alive.resize(cur_n);
        for (int64_t i = 0; i < cur_n; ++i) {                                            // compute_relocation_mask_kernel, :160-203
            const float* m = means + 3 * i; const float* q = quats + 4 * i; const float* s = scales + 3 * i; const float* c = dc + 3 * i;
            const bool low = 1.0f / (1.0f + std::exp(-opacs[i])) <= min_opacity;
            const bool fin = std::isfinite((m[0] * m[0] + m[1] * m[1] + m[2] * m[2]) / (q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]) +
                                           (s[0] * c[0] + s[1] * c[1] + s[2] * c[2]) * opacs[i]);
            alive[i] = !(low || !fin);
            if (!alive[i]) dst.push_back((int32_t)i);
        }
        count = (int64_t)dst.size();
    }
    if (count == 0) return 0;
    std::vector<int32_t> src(count);
    oracle_weighted_sample(cur_n, seed, weights, mode == 0 ? alive.data() : nullptr, count, src.data());
    for (int64_t i = 0; i < count; ++i) {
        const int64_t d = mode == 0 ? dst[i] : cur_n + i;
        split_one(a, src[i], d, split_k);
        if (src_out) src_out[i] = src[i];
        if (dst_out) dst_out[i] = (int32_t)d;
    }
    return count;
}

}  // extern "C"
