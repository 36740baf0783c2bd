// Gaussian projection forward and backward.
//
// Forward: per (view, splat) pair, world mean -> camera, 3D covariance from the
// normalised quaternion and exp(scale), EWA 2D covariance through the camera
// Jacobian, +0.3 px blur, conic, opacity-aware extent, culls, SH degree 3 ->
// RGB (fp32 or q8/q16 packed coefficients).  Restates
// src/shaders/primitive_3dgs.slang:419-578 and
// src/kernels/projection/ProjectionFwd_kernel.cuh:15-111 of the reference.
//
// Backward: hand-derived reverse mode of the same function with every cull
// skipped (the reference differentiates the assume_valid variant,
// src/shaders/primitive_3dgs.slang:644-698) plus the SH vjp with the colour
// clamp mask (src/shaders/harmonics.slang:1087-1126).
//
// Memory plan: one thread per splat; the 45 SH coefficients of a block's 128
// splats are one contiguous 23 KB span, loaded with coalesced 4-byte accesses
// into shared memory (decoded on the way when packed) and read back at stride
// 45 words, which is bank-conflict free.  The backward kernel keeps a second
// 23 KB span for the SH gradients so they too leave the SM coalesced.
#include "ssb_common.cuh"

namespace ssb {

constexpr int kProjBlock = 128;
constexpr int kShPerSplat = 3 * kNumSh;  // 45

struct ProjGeom {
    // forward intermediates kept for the backward pass
    float mc[3];
    float len;
    float opacity;
    float qn[4], qinv;
    float s[3];
    float Rq[9];
    float W[9];       // R * Rq
    float covc[6];    // xx xy xz yy yz zz
    float J00, J02, J11, J12;
    int clampx, clampy;  // -1 below, 0 inside, +1 above
    float Jw[6];         // full 2x3 Jacobian (fisheye, equirectangular)
    float c00, c01, c11, det;
    float mean2d[2];
    float conic[3];
};

__device__ __forceinline__ void quat_to_rot(const float q[4], float R[9]) {
    float w = q[0], x = q[1], y = q[2], z = q[3];
    R[0] = 1.f - 2.f * (y * y + z * z); R[1] = 2.f * (x * y - w * z); R[2] = 2.f * (x * z + w * y);
    R[3] = 2.f * (x * y + w * z); R[4] = 1.f - 2.f * (x * x + z * z); R[5] = 2.f * (y * z - w * x);
    R[6] = 2.f * (x * z - w * y); R[7] = 2.f * (y * z + w * x); R[8] = 1.f - 2.f * (x * x + y * y);
}

// ---- camera models other than pinhole -------------------------------------
// A value with its three partial derivatives with respect to the camera-space
// mean.  The backward pass needs d(Jacobian)/d(mean) of the fisheye and
// equirectangular projections; evaluating the closed-form Jacobian once in this
// arithmetic yields all eighteen second derivatives.
struct D3 { float v, dx, dy, dz; };
__device__ __forceinline__ float val(float a) { return a; }
__device__ __forceinline__ float val(const D3& a) { return a.v; }
__device__ __forceinline__ D3 operator+(const D3& a, const D3& b) { return {a.v + b.v, a.dx + b.dx, a.dy + b.dy, a.dz + b.dz}; }
__device__ __forceinline__ D3 operator-(const D3& a, const D3& b) { return {a.v - b.v, a.dx - b.dx, a.dy - b.dy, a.dz - b.dz}; }
__device__ __forceinline__ D3 operator-(const D3& a) { return {-a.v, -a.dx, -a.dy, -a.dz}; }
__device__ __forceinline__ D3 operator*(const D3& a, const D3& b) {
    return {a.v * b.v, a.dx * b.v + a.v * b.dx, a.dy * b.v + a.v * b.dy, a.dz * b.v + a.v * b.dz};
}
__device__ __forceinline__ D3 operator/(const D3& a, const D3& b) {
    float r = 1.0f / b.v, q = a.v * r;
    return {q, (a.dx - q * b.dx) * r, (a.dy - q * b.dy) * r, (a.dz - q * b.dz) * r};
}
__device__ __forceinline__ D3 operator*(float a, const D3& b) { return {a * b.v, a * b.dx, a * b.dy, a * b.dz}; }
__device__ __forceinline__ D3 operator*(const D3& b, float a) { return a * b; }
__device__ __forceinline__ D3 operator/(float a, const D3& b) { return D3{a, 0.f, 0.f, 0.f} / b; }
__device__ __forceinline__ D3 operator/(const D3& a, float b) { return (1.0f / b) * a; }
__device__ __forceinline__ D3 operator-(float a, const D3& b) { return {a - b.v, -b.dx, -b.dy, -b.dz}; }
__device__ __forceinline__ D3 operator+(float a, const D3& b) { return {a + b.v, b.dx, b.dy, b.dz}; }
__device__ __forceinline__ D3 operator+(const D3& b, float a) { return {a + b.v, b.dx, b.dy, b.dz}; }
__device__ __forceinline__ float sqrt_s(float a) { return sqrtf(a); }
__device__ __forceinline__ D3 sqrt_s(const D3& a) {
    float r = sqrtf(a.v), h = 0.5f / r;
    return {r, a.dx * h, a.dy * h, a.dz * h};
}
__device__ __forceinline__ float atan2_s(float y, float x) { return atan2f(y, x); }
__device__ __forceinline__ D3 atan2_s(const D3& y, const D3& x) {
    float r = 1.0f / (x.v * x.v + y.v * y.v);
    return {atan2f(y.v, x.v), (x.v * y.dx - y.v * x.dx) * r, (x.v * y.dy - y.v * x.dy) * r, (x.v * y.dz - y.v * x.dz) * r};
}
__device__ __forceinline__ float lift(float a, float) { return a; }
__device__ __forceinline__ D3 lift(float a, const D3&) { return {a, 0.f, 0.f, 0.f}; }

// Pixel position and 2x3 Jacobian d(uv)/d(p) of the equidistant fisheye
// (src/shaders/projection_utils.slang:378-384,400-410: k = theta / r, with the
// series (1 - theta^2/3)/z below theta = 1e-3), of the equisolid fisheye (:388-395:
// k = 2 sin(theta/2) / r, written algebraically below) and of the equirectangular
// camera (:505-518: lon = atan2(x, z), lat = atan2(y, hypot(x, z))), as closed
// forms of the derivatives the reference takes by forward-mode autodiff (:463-476, :537-548).
template <int MODEL, class S>
__device__ __forceinline__ void project_mean_wide(const S p[3], float fx, float fy, float cx, float cy, S uv[2], S J[6]) {
    if (MODEL == SSB_CAMERA_FISHEYE) {
        S r2 = p[0] * p[0] + p[1] * p[1];
        S r = sqrt_s(r2);
        S theta = atan2_s(r, p[2]);
        S rho2 = r2 + p[2] * p[2];
        S k, dkx, dky, dkz;
        S dtz = -(r / rho2);
        if (val(theta) < 1e-3f) {
            k = (1.0f - theta * theta * (1.0f / 3.0f)) / p[2];
            S rinv = val(r) > 0.f ? 1.0f / r : lift(0.f, r);
            S dtx = p[2] * p[0] * rinv / rho2, dty = p[2] * p[1] * rinv / rho2;
            S c = (-(2.0f / 3.0f)) * theta / p[2];
            dkx = c * dtx; dky = c * dty; dkz = c * dtz - k / p[2];
        } else {
            k = theta / r;
            S ir = 1.0f / r;
            S dtx = p[2] * p[0] / (r * rho2), dty = p[2] * p[1] / (r * rho2);
            S tir3 = theta * ir * ir * ir;
            dkx = dtx * ir - tir3 * p[0];
            dky = dty * ir - tir3 * p[1];
            dkz = dtz * ir;
        }
        uv[0] = fx * (p[0] * k) + lift(cx, k);
        uv[1] = fy * (p[1] * k) + lift(cy, k);
        J[0] = fx * (k + p[0] * dkx); J[1] = fx * (p[0] * dky); J[2] = fx * (p[0] * dkz);
        J[3] = fy * (p[1] * dkx); J[4] = fy * (k + p[1] * dky); J[5] = fy * (p[1] * dkz);
    } else if (MODEL == SSB_CAMERA_EQUISOLID) {
        // 2 sin(theta/2) / r = sqrt(2 / (rho (rho + z))), rho = |p|: one algebraic form for every r, free of
        // the cancellation in the derivative of the trigonometric one; rho + z = r^2 / (rho - z) behind the camera
        S r2 = p[0] * p[0] + p[1] * p[1];
        S rho2 = r2 + p[2] * p[2];
        S rho = sqrt_s(rho2);
        S w = val(p[2]) >= 0.f ? rho + p[2] : r2 / (rho - p[2]);
        S q = rho * w;
        S k = sqrt_s(2.0f / q);
        S c = -(k / (2.0f * q * rho));
        S t = 2.0f * rho + p[2];
        S dkx = c * (p[0] * t), dky = c * (p[1] * t);
        S dkz = -(k * w / (2.0f * rho2));
        uv[0] = fx * (p[0] * k) + lift(cx, k);
        uv[1] = fy * (p[1] * k) + lift(cy, k);
        J[0] = fx * (k + p[0] * dkx); J[1] = fx * (p[0] * dky); J[2] = fx * (p[0] * dkz);
        J[3] = fy * (p[1] * dkx); J[4] = fy * (k + p[1] * dky); J[5] = fy * (p[1] * dkz);
    } else if (MODEL == SSB_CAMERA_PINHOLE) {
        // only reached with a lens distortion tier (the undistorted pinhole has its own sparse-Jacobian path)
        S rz = 1.0f / p[2];
        S u = p[0] * rz, v = p[1] * rz;
        uv[0] = fx * u + lift(cx, u);
        uv[1] = fy * v + lift(cy, v);
        J[0] = fx * rz; J[1] = lift(0.f, rz); J[2] = -((fx * u) * rz);
        J[3] = lift(0.f, rz); J[4] = fy * rz; J[5] = -((fy * v) * rz);
    } else {
        S h2 = p[0] * p[0] + p[2] * p[2];
        S h = sqrt_s(h2);
        uv[0] = fx * atan2_s(p[0], p[2]) + lift(cx, h);
        uv[1] = fy * atan2_s(p[1], h) + lift(cy, h);
        S rho2 = h2 + p[1] * p[1];
        S hr = h * rho2;
        J[0] = fx * (p[2] / h2); J[1] = lift(0.f, h); J[2] = fx * (-(p[0] / h2));
        J[3] = fy * (-(p[1] * p[0]) / hr); J[4] = fy * (h / rho2); J[5] = fy * (-(p[1] * p[2]) / hr);
    }
}

// ---- lens distortion tiers -------------------------------------------------
// The reference's three tiers (src/shaders/projection_utils.slang:242-298) are special cases of one map of the camera
// model's normalised coordinates:
//   radial = (1 + r2 (n1 + r2 (n2 + r2 (n3 + r2 n4)))) / (1 + r2 (d1 + r2 (d2 + r2 d3)))
//   u' = u radial + 2 p1 u v + p2 (r2 + 2 u^2) + s1 r2,   v' = v radial + 2 p2 u v + p1 (r2 + 2 v^2) + s2 r2
// OpenCV: n1 n2 p1 p2.  Thin prism: n1..n4 p1 p2 s1 s2.  Rational: n1..n3, d1..d3, p1 p2.  Unused terms are zero, which
// leaves the tier's own arithmetic (x + 0, x / 1).  Each tier's coefficient row has its own order (:246,:262,:283).
struct LensDist { float n1, n2, n3, n4, d1, d2, d3, p1, p2, s1, s2; };
struct DistArgs { const float* coeffs; int tier; int n_sh; };   // [C][8] rows (NULL reads as zeros), SSB_DISTORTION_*; SH coefficients past DC in use

__device__ __forceinline__ LensDist load_lens(const DistArgs& da, int cid) {
    LensDist k = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (da.coeffs == nullptr) return k;
    const float* c = da.coeffs + 8 * cid;
    if (da.tier == SSB_DISTORTION_OPENCV) { k.n1 = c[0]; k.n2 = c[1]; k.p1 = c[2]; k.p2 = c[3]; }
    else if (da.tier == SSB_DISTORTION_THIN_PRISM) { k.n1 = c[0]; k.n2 = c[1]; k.n3 = c[2]; k.n4 = c[3]; k.p1 = c[4]; k.p2 = c[5]; k.s1 = c[6]; k.s2 = c[7]; }
    else { k.n1 = c[0]; k.n2 = c[1]; k.n3 = c[2]; k.d1 = c[3]; k.d2 = c[4]; k.d3 = c[5]; k.p1 = c[6]; k.p2 = c[7]; }
    return k;
}

// The distorted point and the 2x2 Jacobian of the map (row major), as closed forms of what the reference takes by
// forward-mode autodiff (camera_distortion_jac, :300-308)
template <class S>
__device__ __forceinline__ void distort_s(const LensDist& k, const S& u, const S& v, S out[2], S Dj[4]) {
    S uu = u * u, vv = v * v, uv = u * v;
    S r2 = uu + vv;
    S num = 1.0f + r2 * (k.n1 + r2 * (k.n2 + r2 * (k.n3 + k.n4 * r2)));
    S den = 1.0f + r2 * (k.d1 + r2 * (k.d2 + k.d3 * r2));
    S dnum = k.n1 + r2 * (2.0f * k.n2 + r2 * (3.0f * k.n3 + (4.0f * k.n4) * r2));
    S dden = k.d1 + r2 * (2.0f * k.d2 + (3.0f * k.d3) * r2);
    S radial = num / den;
    S drad = (dnum - radial * dden) / den;          // d radial / d r2
    S ru = (2.0f * drad) * u, rv = (2.0f * drad) * v;
    out[0] = u * radial + ((2.0f * k.p1) * uv + k.p2 * (r2 + 2.0f * uu) + k.s1 * r2);
    out[1] = v * radial + ((2.0f * k.p2) * uv + k.p1 * (r2 + 2.0f * vv) + k.s2 * r2);
    Dj[0] = radial + u * ru + ((2.0f * k.p1) * v + (6.0f * k.p2 + 2.0f * k.s1) * u);
    Dj[1] = u * rv + ((2.0f * k.p1) * u + (2.0f * k.p2 + 2.0f * k.s1) * v);
    Dj[2] = v * ru + ((2.0f * k.p2) * v + (2.0f * k.p1 + 2.0f * k.s2) * u);
    Dj[3] = radial + v * rv + ((2.0f * k.p2) * u + (6.0f * k.p1 + 2.0f * k.s2) * v);
}

// is_valid_distortion (:311-323)
__device__ __forceinline__ bool lens_valid(const LensDist& k, float u, float v) {
    float out[2], Dj[4];
    distort_s<float>(k, u, v, out, Dj);
    float jdet = fminf(Dj[0] * Dj[3] - Dj[1] * Dj[2], fminf(Dj[0], Dj[3]));
    return jdet > 0.25f && jdet < 4.0f && (u * out[0] + v * out[1]) >= 0.0f;
}

// Pixel position and 2x3 Jacobian with a distortion tier: uv = f * distort(n(p)) + c, J = diag(f) Dj dn/dp
// (persp_proj_uv / fisheye_proj_uv / equisolid_proj_uv and their Jacobians, :330-343,363-375,412-424,443-493); for the
// pinhole the third column is then limited as in persp_proj_3dgs (src/shaders/primitive_3dgs.slang:84-95), the limits
// carrying their own dependence on z.  n_out receives the normalised coordinates.
template <int MODEL, class S>
__device__ __forceinline__ void project_mean_dist(const S p[3], const CamDev& cam, const LensDist& k, int W_img, S uv[2], S J[6], S n_out[2]) {
    S Jn[6];
    project_mean_wide<MODEL, S>(p, 1.0f, 1.0f, 0.0f, 0.0f, n_out, Jn);
    S d[2], Dj[4];
    distort_s<S>(k, n_out[0], n_out[1], d, Dj);
    uv[0] = cam.fx * d[0] + lift(cam.cx, d[0]);
    uv[1] = cam.fy * d[1] + lift(cam.cy, d[1]);
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        J[j] = cam.fx * (Dj[0] * Jn[j] + Dj[1] * Jn[3 + j]);
        J[3 + j] = cam.fy * (Dj[2] * Jn[j] + Dj[3] * Jn[3 + j]);
    }
    if (MODEL == SSB_CAMERA_PINHOLE) {
        float width = (float)W_img;
        float lim_pos = width + 0.3f * (0.5f * width), lim_neg = 0.3f * (0.5f * width);
        S rz = 1.0f / p[2];
        S max_x = (lim_neg + cam.cx) * rz, min_x = -((lim_pos - cam.cx) * rz);
        S max_y = (lim_neg + cam.cy) * rz, min_y = -((lim_pos - cam.cy) * rz);
        if (val(J[2]) < val(min_x)) J[2] = min_x; else if (val(J[2]) > val(max_x)) J[2] = max_x;
        if (val(J[5]) < val(min_y)) J[5] = min_y; else if (val(J[5]) > val(max_y)) J[5] = max_y;
    }
}

// Geometry of the projection.  Returns false when a cull of the reference's
// forward pass applies (never when assume_valid).
template <int MODEL, bool DIST, bool assume_valid>
__device__ __forceinline__ bool project_geom(
    const CamDev& cam, const LensDist& lens, int W_img, bool antialiased,
    const float mean[3], const float quat[4], const float scale[3], float in_opacity,
    ProjGeom& g) {
    const float* R = cam.R;
#pragma unroll
    for (int i = 0; i < 3; ++i) g.mc[i] = R[3 * i] * mean[0] + R[3 * i + 1] * mean[1] + R[3 * i + 2] * mean[2] + cam.t[i];
    g.len = sqrtf(g.mc[0] * g.mc[0] + g.mc[1] * g.mc[1] + g.mc[2] * g.mc[2]);
    if (!assume_valid && (MODEL == SSB_CAMERA_PINHOLE ? g.mc[2] : g.len) <= 0.0f) return false;
    g.opacity = 1.0f / (1.0f + expf(-in_opacity));

    float qq = sqrtf(quat[0] * quat[0] + quat[1] * quat[1] + quat[2] * quat[2] + quat[3] * quat[3]);
    g.qinv = 1.0f / qq;
#pragma unroll
    for (int i = 0; i < 4; ++i) g.qn[i] = quat[i] * g.qinv;
    quat_to_rot(g.qn, g.Rq);
#pragma unroll
    for (int i = 0; i < 3; ++i) g.s[i] = expf(scale[i]);
    // W = R * Rq ; covc = W diag(s^2) W^T
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
        for (int j = 0; j < 3; ++j)
            g.W[3 * i + j] = R[3 * i] * g.Rq[j] + R[3 * i + 1] * g.Rq[3 + j] + R[3 * i + 2] * g.Rq[6 + j];
    float s2[3] = {g.s[0] * g.s[0], g.s[1] * g.s[1], g.s[2] * g.s[2]};
    const float* Wm = g.W;
    g.covc[0] = Wm[0] * Wm[0] * s2[0] + Wm[1] * Wm[1] * s2[1] + Wm[2] * Wm[2] * s2[2];
    g.covc[1] = Wm[0] * Wm[3] * s2[0] + Wm[1] * Wm[4] * s2[1] + Wm[2] * Wm[5] * s2[2];
    g.covc[2] = Wm[0] * Wm[6] * s2[0] + Wm[1] * Wm[7] * s2[1] + Wm[2] * Wm[8] * s2[2];
    g.covc[3] = Wm[3] * Wm[3] * s2[0] + Wm[4] * Wm[4] * s2[1] + Wm[5] * Wm[5] * s2[2];
    g.covc[4] = Wm[3] * Wm[6] * s2[0] + Wm[4] * Wm[7] * s2[1] + Wm[5] * Wm[8] * s2[2];
    g.covc[5] = Wm[6] * Wm[6] * s2[0] + Wm[7] * Wm[7] * s2[1] + Wm[8] * Wm[8] * s2[2];

    float c00, c01, c11;
    const float* c = g.covc;
    if (MODEL == SSB_CAMERA_PINHOLE && !DIST) {
        float rz = 1.0f / g.mc[2];
        float u = g.mc[0] * rz, v = g.mc[1] * rz;
        g.mean2d[0] = cam.fx * u + cam.cx;
        g.mean2d[1] = cam.fy * v + cam.cy;
        g.J00 = cam.fx * rz;
        g.J11 = cam.fy * rz;
        float j02 = -(cam.fx * u) * rz, j12 = -(cam.fy * v) * rz;
        // Both rows use the x limits, as the reference does
        // (src/shaders/primitive_3dgs.slang:84-95).
        float width = (float)W_img;
        float lim_pos = width + 0.3f * (0.5f * width);
        float lim_neg = 0.3f * (0.5f * width);
        float max_x = -(-lim_neg - cam.cx) * rz, min_x = -(lim_pos - cam.cx) * rz;
        float max_y = -(-lim_neg - cam.cy) * rz, min_y = -(lim_pos - cam.cy) * rz;
        g.clampx = j02 < min_x ? -1 : (j02 > max_x ? 1 : 0);
        g.clampy = j12 < min_y ? -1 : (j12 > max_y ? 1 : 0);
        g.J02 = g.clampx < 0 ? min_x : (g.clampx > 0 ? max_x : j02);
        g.J12 = g.clampy < 0 ? min_y : (g.clampy > 0 ? max_y : j12);

        // cov2d = J covc J^T with J = [[J00, 0, J02], [0, J11, J12]]
        float a0 = g.J00 * c[0] + g.J02 * c[2], a1 = g.J00 * c[1] + g.J02 * c[4], a2 = g.J00 * c[2] + g.J02 * c[5];
        float b1 = g.J11 * c[3] + g.J12 * c[4], b2 = g.J11 * c[4] + g.J12 * c[5];
        c00 = a0 * g.J00 + a2 * g.J02;
        c01 = a1 * g.J11 + a2 * g.J12;
        c11 = b1 * g.J11 + b2 * g.J12;
    } else {
        if (DIST) {
            float nrm[2];
            project_mean_dist<MODEL, float>(g.mc, cam, lens, W_img, g.mean2d, g.Jw, nrm);
            // persp_proj / fisheye_proj / equisolid_proj: a point where the distortion map folds is dropped (:346-358,427-441)
            if (!assume_valid && !lens_valid(lens, nrm[0], nrm[1])) return false;
        } else {
            project_mean_wide<MODEL, float>(g.mc, cam.fx, cam.fy, cam.cx, cam.cy, g.mean2d, g.Jw);
        }
        const float* J = g.Jw;
        // rows of J covc (covc symmetric: xx xy xz yy yz zz)
        float a0 = J[0] * c[0] + J[1] * c[1] + J[2] * c[2], a1 = J[0] * c[1] + J[1] * c[3] + J[2] * c[4], a2 = J[0] * c[2] + J[1] * c[4] + J[2] * c[5];
        float b0 = J[3] * c[0] + J[4] * c[1] + J[5] * c[2], b1 = J[3] * c[1] + J[4] * c[3] + J[5] * c[4], b2 = J[3] * c[2] + J[4] * c[4] + J[5] * c[5];
        c00 = a0 * J[0] + a1 * J[1] + a2 * J[2];
        c01 = a0 * J[3] + a1 * J[4] + a2 * J[5];
        c11 = b0 * J[3] + b1 * J[4] + b2 * J[5];
        if (!assume_valid && (MODEL == SSB_CAMERA_FISHEYE || MODEL == SSB_CAMERA_EQUISOLID)) {
            // behind-the-camera splats that still reach the image centre are dropped
            // (src/shaders/primitive_3dgs.slang:515-521); c10 == c01 here
            float invd = 1.0f / (c00 * c11 - c01 * c01);
            float mx = g.mean2d[0] - cam.cx, my = g.mean2d[1] - cam.cy;
            float q = (c11 * invd * mx - c01 * invd * my) * mx + (-c01 * invd * mx + c00 * invd * my) * my;
            float opac = g.opacity * expf(-0.5f * q);
            if (g.mc[2] < 0.0f && opac > kAlphaThreshold) return false;
        }
    }
    const float eps2d = antialiased ? 0.1f : 0.3f;
    float det_orig = c00 * c11 - c01 * c01;
    c00 += eps2d; c11 += eps2d;
    float det = c00 * c11 - c01 * c01;
    if (!assume_valid && det <= 0.f) return false;
    g.c00 = c00; g.c01 = c01; g.c11 = c11; g.det = det;
    float invdet = 1.0f / det;
    g.conic[0] = c11 * invdet; g.conic[1] = -c01 * invdet; g.conic[2] = c00 * invdet;
    if (antialiased) g.opacity *= sqrtf(fmaxf(0.f, det_orig / det));
    if (!assume_valid && g.opacity < kAlphaThreshold) return false;
    return true;
}

// Real SH basis, bands 1..3, at a unit direction (src/shaders/harmonics.slang:154-251).
__device__ __forceinline__ void sh_basis(float x, float y, float z, float b[kNumSh]) {
    const float c1 = 0.48860251190292f;
    b[0] = -c1 * y; b[1] = c1 * z; b[2] = -c1 * x;
    float z2 = z * z;
    float t0b = -1.092548430592079f * z;
    const float c2a = 0.5462742152960395f;
    float fC1 = x * x - y * y, fS1 = 2.f * x * y;
    b[3] = c2a * fS1; b[4] = t0b * y; b[5] = 0.9461746957575601f * z2 - 0.3153915652525201f;
    b[6] = t0b * x; b[7] = c2a * fC1;
    float t0c = -2.285228997322329f * z2 + 0.4570457994644658f;
    float t1b = 1.445305721320277f * z;
    const float c3a = -0.5900435899266435f;
    float fC2 = x * fC1 - y * fS1, fS2 = x * fS1 + y * fC1;
    b[8] = c3a * fS2; b[9] = t1b * fS1; b[10] = t0c * y;
    b[11] = z * (1.865881662950577f * z2 - 1.119528997770346f);
    b[12] = t0c * x; b[13] = t1b * fC1; b[14] = c3a * fC2;
}

// Loads the block's SH span into shared memory as fp32 (decoding packed codes).
// A full block's span starts on a 16-byte boundary in every format (128 * 45 cells), so it is
// brought in with 16-byte asynchronous copies (global -> shared without passing through
// registers, all of a thread's copies in flight at once): fp32 coefficients straight into
// sh_s, packed codes into raw_s, from where they are decoded 8 (16-bit) or 16 (8-bit) at a
// time -- the codes of one vector share a bounds entry whenever the bounds stride is a
// multiple of the vector's cell count.  Register-staged 16-byte loads were measured slower
// than 4-byte ones here; the asynchronous copies are a quarter faster than either.
// Partial blocks and unaligned arrays take 4-byte loads.
__device__ __forceinline__ void async_copy_span(void* smem_dst, const void* gmem_src, int n_vec16) {
    const uint32_t sdst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const uint4* src = (const uint4*)gmem_src;
    for (int v = threadIdx.x; v < n_vec16; v += kProjBlock)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sdst + 16u * (uint32_t)v), "l"(src + v) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void async_copy_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kShRawBytes = kProjBlock * kShPerSplat * 2;   // a block's 16-bit codes

__device__ __forceinline__ void stage_sh(
    float* sh_s, unsigned char* raw_s, const float* __restrict__ sh_f32, const void* __restrict__ packed, const float* __restrict__ bounds,
    int bits, int64_t bounds_stride, int64_t first_splat, int64_t n) {
    const int64_t base = first_splat * kShPerSplat;
    const int count = (int)min((int64_t)kProjBlock, n - first_splat) * kShPerSplat;
    const bool quant = bits == 8 || bits == 16;
    const void* arr = quant ? packed : (const void*)sh_f32;
    const bool full = count == kProjBlock * kShPerSplat && ((uintptr_t)arr & 15) == 0;
    if (full && !quant) {
        async_copy_span(sh_s, sh_f32 + base, kProjBlock * kShPerSplat / 4);
        async_copy_wait();
    } else if (full && bits == 16 && (bounds_stride & 7) == 0) {
        async_copy_span(raw_s, (const uint16_t*)packed + base, kProjBlock * kShPerSplat / 8);
        const int64_t b0 = base / bounds_stride;
        const unsigned r0 = (unsigned)(base - b0 * bounds_stride), stride = (unsigned)min(bounds_stride, (int64_t)0x7fffffff);
        const float inv = 1.0f / 65535.0f;
        async_copy_wait();
        __syncthreads();
        for (int v = threadIdx.x; v < kProjBlock * kShPerSplat / 8; v += kProjBlock) {
            const uint4 c = ((const uint4*)raw_s)[v];
            const float2 mm = ((const float2*)bounds)[b0 + (r0 + 8u * v) / stride];
            const float d = mm.y - mm.x;
            float4 lo, hi;
            lo.x = mm.x + d * ((float)(c.x & 0xffffu) * inv); lo.y = mm.x + d * ((float)(c.x >> 16) * inv);
            lo.z = mm.x + d * ((float)(c.y & 0xffffu) * inv); lo.w = mm.x + d * ((float)(c.y >> 16) * inv);
            hi.x = mm.x + d * ((float)(c.z & 0xffffu) * inv); hi.y = mm.x + d * ((float)(c.z >> 16) * inv);
            hi.z = mm.x + d * ((float)(c.w & 0xffffu) * inv); hi.w = mm.x + d * ((float)(c.w >> 16) * inv);
            ((float4*)sh_s)[2 * v] = lo; ((float4*)sh_s)[2 * v + 1] = hi;
        }
    } else if (full && bits == 8 && (bounds_stride & 15) == 0) {
        async_copy_span(raw_s, (const uint8_t*)packed + base, kProjBlock * kShPerSplat / 16);
        const int64_t b0 = base / bounds_stride;
        const unsigned r0 = (unsigned)(base - b0 * bounds_stride), stride = (unsigned)min(bounds_stride, (int64_t)0x7fffffff);
        const float inv = 1.0f / 255.0f;
        async_copy_wait();
        __syncthreads();
        for (int v = threadIdx.x; v < kProjBlock * kShPerSplat / 16; v += kProjBlock) {
            const uint4 c = ((const uint4*)raw_s)[v];
            const float2 mm = ((const float2*)bounds)[b0 + (r0 + 16u * v) / stride];
            const float d = mm.y - mm.x;
            const unsigned w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float4 o;
                o.x = mm.x + d * ((float)(w[k] & 0xffu) * inv); o.y = mm.x + d * ((float)((w[k] >> 8) & 0xffu) * inv);
                o.z = mm.x + d * ((float)((w[k] >> 16) & 0xffu) * inv); o.w = mm.x + d * ((float)(w[k] >> 24) * inv);
                ((float4*)sh_s)[4 * v + k] = o;
            }
        }
    } else if (quant) {
        const float inv = bits == 8 ? (1.0f / 255.0f) : (1.0f / 65535.0f);
        for (int i = threadIdx.x; i < count; i += kProjBlock) {
            int64_t cell = base + i;
            float q = bits == 8 ? (float)((const uint8_t*)packed)[cell] : (float)((const uint16_t*)packed)[cell];
            float2 mm = ((const float2*)bounds)[cell / bounds_stride];
            sh_s[i] = mm.x + (mm.y - mm.x) * (q * inv);
        }
    } else {
        for (int i = threadIdx.x; i < count; i += kProjBlock) sh_s[i] = sh_f32[base + i];
    }
}

// PACK = 0: one output slot per (view, splat) pair, culled pairs marked by an all-zero box.
// PACK = 1: the visibility pass of the packed projection: only flags[pair] = kept (no SH, no other output).
// PACK = 2: its compacting pass: a kept pair goes to slot flags[pair] (by then the exclusive scan of the flags), with its
//           view and splat index; culled pairs write nothing; slots beyond `capacity` are dropped.
struct PackArgs {
    int32_t* flags;          // [views * n]
    int32_t* camera_ids;     // [capacity]
    int32_t* gaussian_ids;   // [capacity]
    int64_t capacity;
};

template <int MODEL, int PACK, bool DIST>
__global__ void __launch_bounds__(kProjBlock) project_fwd_kernel(
    SsbSplats sp, SsbShQuant shq, int64_t n, const float* __restrict__ viewmats, const float* __restrict__ intrins,
    int W, int H, int antialiased,
    float4* __restrict__ aabb_out, float* __restrict__ depths_out, float* __restrict__ radii, SsbScreenRec* __restrict__ screen, PackArgs pk,
    DistArgs da) {
    __shared__ __align__(16) float sh_s[PACK == 1 ? 4 : kProjBlock * kShPerSplat];
    __shared__ __align__(16) unsigned char raw_s[PACK == 1 ? 16 : kShRawBytes];
    const int cid = blockIdx.y;
    const int64_t first = (int64_t)blockIdx.x * kProjBlock;
    const int64_t gid = first + threadIdx.x;
    // per-splat loads are issued before the SH span is staged, so both are in flight together
    const int64_t gl = gid < n ? gid : n - 1;
    float mean[3] = {sp.means[3 * gl], sp.means[3 * gl + 1], sp.means[3 * gl + 2]};
    float4 q4 = ((const float4*)sp.quats)[gl];
    float quat[4] = {q4.x, q4.y, q4.z, q4.w};
    float scale[3] = {sp.scales[3 * gl], sp.scales[3 * gl + 1], sp.scales[3 * gl + 2]};
    float in_op = sp.opacities[gl];
    float dc_in[3] = {sp.features_dc[3 * gl], sp.features_dc[3 * gl + 1], sp.features_dc[3 * gl + 2]};
    CamDev cam = load_cam(viewmats, intrins, cid);
    if (PACK != 1) {
        stage_sh(sh_s, raw_s, sp.features_sh, shq.packed, shq.bounds, shq.bits, shq.bounds_stride, first, n);
        __syncthreads();
    }
    if (gid >= n) return;
    int64_t idx = (int64_t)cid * n + gid;

    ProjGeom g;
    LensDist lens = {};
    if (DIST) lens = load_lens(da, cid);
    bool ok = project_geom<MODEL, DIST, false>(cam, lens, W, antialiased != 0, mean, quat, scale, in_op, g);
    float xmin = 0.f, ymin = 0.f, xmax = 0.f, ymax = 0.f, L = 0.f;
    if (ok) {
        L = logf(g.opacity / kAlphaThreshold);
        float extend = fminf(3.33f, sqrtf(2.0f * L));
        float rx = extend * sqrtf(g.c00), ry = extend * sqrtf(g.c11);
        xmin = g.mean2d[0] - rx; xmax = g.mean2d[0] + rx;
        ymin = g.mean2d[1] - ry; ymax = g.mean2d[1] + ry;
        if (xmax <= 0.f || xmin >= (float)W || ymax <= 0.f || ymin >= (float)H) ok = false;
    }
    float rgb[3] = {0.f, 0.f, 0.f};
    if (PACK != 1 && ok && xmax > xmin && ymax > ymin) {
        // viewdir = mean + R^T t, normalised inside the SH evaluation
        const float* R = cam.R;
        float d[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) d[j] = mean[j] + (R[j] * cam.t[0] + R[3 + j] * cam.t[1] + R[6 + j] * cam.t[2]);
        float inv = rsqrtf(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
        float b[kNumSh];
        sh_basis(d[0] * inv, d[1] * inv, d[2] * inv, b);
        const float* sh = sh_s + threadIdx.x * kShPerSplat;
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
            float c = kShC0 * dc_in[ch];
#pragma unroll
            for (int j = 0; j < kNumSh; ++j) if (j < da.n_sh) c += b[j] * sh[3 * j + ch];     // bands above the active degree are not read
            rgb[ch] = fmaxf(c + 0.5f, 0.0f);
        }
    }
    float a0 = fminf(fmaxf(xmin, 0.0f), (float)W - 1.0f), a1 = fminf(fmaxf(ymin, 0.0f), (float)H - 1.0f);
    float a2 = fminf(fmaxf(xmax, 0.0f), (float)W - 1.0f), a3 = fminf(fmaxf(ymax, 0.0f), (float)H - 1.0f);
    bool keep = ok && (a2 - a0 > 1e-3f) && (a3 - a1 > 1e-3f);
    if (PACK == 1) { pk.flags[idx] = keep ? 1 : 0; return; }
    if (PACK == 2) {
        if (!keep) return;
        const int64_t slot = pk.flags[idx];
        if (slot >= pk.capacity) return;
        pk.camera_ids[slot] = cid;
        pk.gaussian_ids[slot] = (int32_t)gid;
        idx = slot;
    }
    if (keep) {
        aabb_out[idx] = make_float4(a0, a1, a2, a3);
        // sorting depth (src/shaders/projection_utils.slang:1012-1029): z for pinhole, squared
        // distance for equirectangular, z^4 + (x^2+y^2)^2/512 for fisheye
        float sd;
        if (MODEL == SSB_CAMERA_PINHOLE) sd = g.mc[2];
        else if (MODEL == SSB_CAMERA_EQUIRECT) sd = g.mc[0] * g.mc[0] + g.mc[1] * g.mc[1] + g.mc[2] * g.mc[2];
        else {
            float xy2 = g.mc[0] * g.mc[0] + g.mc[1] * g.mc[1];
            sd = g.mc[2] * g.mc[2] * g.mc[2] * g.mc[2] + (1.0f / 512.0f) * xy2 * xy2;
        }
        depths_out[idx] = sd;
        // half extents of the alpha >= 1/255 footprint, slightly inflated
        float e = sqrtf(2.0f * L) * 1.0005f;
        float hx = e * sqrtf(g.c00) + 1e-3f, hy = e * sqrtf(g.c11) + 1e-3f;
        float4* r = (float4*)(screen + idx);
        r[0] = make_float4(g.mean2d[0], g.mean2d[1], hx, hy);
        r[1] = make_float4(g.conic[0], g.conic[1], g.conic[2], g.opacity);
        r[2] = make_float4(rgb[0], rgb[1], rgb[2], g.len);
        if (radii) {
            // view_radius_3dgs, src/shaders/projection_utils.slang:1033-1043
            const float* R = cam.R;
            float cp[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) cp[j] = -(R[j] * cam.t[0] + R[3 + j] * cam.t[1] + R[6 + j] * cam.t[2]);
            float ext = sqrtf(2.0f * logf(fmaxf(255.0f / (1.0f + expf(-in_op)), 1.0f)));
            float rad = expf(fmaxf(scale[0], fmaxf(scale[1], scale[2]))) * ext;
            float dx = mean[0] - cp[0], dy = mean[1] - cp[1], dz = mean[2] - cp[2];
            float dist = sqrtf(dx * dx + dy * dy + dz * dz);
            float vr = rad / (fmaxf(dist, rad) + sqrtf(fmaxf(dist * dist - rad * rad, 0.0f)));
            atomicMax((int*)&radii[gid], __float_as_int(vr));  // vr >= 0: int order == float order
        }
    } else {
        aabb_out[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
        depths_out[idx] = 0.f;
    }
}

}  // namespace ssb

namespace ssb {

// Gradient of the SH basis with respect to the (unit) direction, contracted
// with the per-coefficient weights w[j] = sum_ch sh[j][ch] * vc[ch].
__device__ __forceinline__ void sh_basis_vjp(float x, float y, float z, const float w[kNumSh], float v[3]) {
    const float c1 = 0.48860251190292f, c2a = 0.5462742152960395f, c2b = 1.092548430592079f;
    const float c3a = -0.5900435899266435f, c3b = 1.445305721320277f, c3c = 2.285228997322329f;
    float z2 = z * z;
    float t0c = -c3c * z2 + 0.4570457994644658f;
    float fC1 = x * x - y * y, fS1 = 2.f * x * y;
    float vx = -c1 * w[2], vy = -c1 * w[0], vz = c1 * w[1];
    vx += 2.f * c2a * y * w[3] - c2b * z * w[6] + 2.f * c2a * x * w[7];
    vy += 2.f * c2a * x * w[3] - c2b * z * w[4] - 2.f * c2a * y * w[7];
    vz += -c2b * y * w[4] + 2.f * 0.9461746957575601f * z * w[5] - c2b * x * w[6];
    vx += c3a * 3.f * fS1 * w[8] + 2.f * c3b * y * z * w[9] + t0c * w[12] + 2.f * c3b * z * x * w[13] + c3a * 3.f * fC1 * w[14];
    vy += c3a * 3.f * fC1 * w[8] + 2.f * c3b * x * z * w[9] + t0c * w[10] - 2.f * c3b * z * y * w[13] - c3a * 3.f * fS1 * w[14];
    vz += c3b * fS1 * w[9] - 2.f * c3c * z * y * w[10] + (3.f * 1.865881662950577f * z2 - 1.119528997770346f) * w[11]
        - 2.f * c3c * z * x * w[12] + c3b * fC1 * w[13];
    v[0] = vx; v[1] = vy; v[2] = vz;
}

__device__ __forceinline__ float finite_or_zero(float v) { return isfinite(v) ? v : 0.0f; }

template <bool MULTI_VIEW, int MODEL, bool DIST>
__global__ void __launch_bounds__(kProjBlock, DIST ? 3 : 4) project_bwd_kernel(
    SsbSplats sp, SsbShQuant shq, int64_t n, int C, const float* __restrict__ viewmats, const float* __restrict__ intrins,
    int W, int H, int antialiased, const float4* __restrict__ aabb, SsbScreenRec* __restrict__ v_screen,
    SsbSplats gr, int accumulate, int clear_v_screen, const int32_t* __restrict__ pair_of, int64_t range_first, int64_t range_end, DistArgs da) {
    // The launch covers splats [range_first, range_end) of the n per view; every array, the gradient arrays included, is
    // indexed by the splat's own number (a caller that keeps gradients for the range only passes pointers moved back by
    // the range's start).
    // pair_of (packed input): aabb and v_screen hold one entry per VISIBLE pair, and pair_of[view * n + splat] is that
    // pair's position, or negative when the pair was culled.  Null: one entry per (view, splat) pair.
    // One view per launch (the training loop's case): a thread's SH gradients overwrite its own
    // SH values in shared memory once they have been read, so one 23 KB span is enough and six
    // CTAs fit an SM.  Several views: gradients accumulate in a second span.
    __shared__ __align__(16) float sh_s[kProjBlock * kShPerSplat];
    __shared__ __align__(16) float shg_multi[MULTI_VIEW ? kProjBlock * kShPerSplat : 4];
    // packed codes land here before they are decoded; with several views the gradient span is still unused then
    __shared__ __align__(16) unsigned char raw_single[MULTI_VIEW ? 16 : kShRawBytes];
    unsigned char* raw_s = MULTI_VIEW ? (unsigned char*)shg_multi : raw_single;
    float* shg_s = MULTI_VIEW ? shg_multi : sh_s;
    const int64_t first = range_first + (int64_t)blockIdx.x * kProjBlock;
    const int64_t gid = first + threadIdx.x;
    const int count = (int)min((int64_t)kProjBlock, range_end - first) * kShPerSplat;
    // per-splat loads (and, for a single view, its aabb and gradient record) are issued before
    // the SH span is staged, so both groups of loads are in flight together
    const int64_t gl = gid < range_end ? gid : range_end - 1;
    float mean[3] = {sp.means[3 * gl], sp.means[3 * gl + 1], sp.means[3 * gl + 2]};
    float4 q4 = ((const float4*)sp.quats)[gl];
    float quat[4] = {q4.x, q4.y, q4.z, q4.w};
    float scale[3] = {sp.scales[3 * gl], sp.scales[3 * gl + 1], sp.scales[3 * gl + 2]};
    float in_op = sp.opacities[gl];
    float dc_in[3] = {sp.features_dc[3 * gl], sp.features_dc[3 * gl + 1], sp.features_dc[3 * gl + 2]};
    const int64_t slot0 = pair_of ? (int64_t)pair_of[gl] : gl;
    float4 bb0 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 vr0[3] = {bb0, bb0, bb0};
    if (slot0 >= 0) {
        bb0 = aabb[slot0];
        const float4* vr = (const float4*)(v_screen + slot0);
        vr0[0] = vr[0]; vr0[1] = vr[1]; vr0[2] = vr[2];
    }
    stage_sh(sh_s, raw_s, sp.features_sh, shq.packed, shq.bounds, shq.bits, shq.bounds_stride, first, range_end);
    if (MULTI_VIEW) {
        __syncthreads();      // every thread is done reading the codes
        for (int i = threadIdx.x; i < count; i += kProjBlock) shg_s[i] = 0.f;
    }
    __syncthreads();
    bool any_view = false;

    float g_mean[3] = {0.f, 0.f, 0.f}, g_quat[4] = {0.f, 0.f, 0.f, 0.f}, g_scale[3] = {0.f, 0.f, 0.f}, g_op = 0.f, g_dc[3] = {0.f, 0.f, 0.f};
    if (gid < range_end) {
        const float* sh = sh_s + threadIdx.x * kShPerSplat;
        float* shg = shg_s + threadIdx.x * kShPerSplat;
        for (int cid = 0; cid < C; ++cid) {
            const int64_t lin = (int64_t)cid * n + gid;
            const int64_t idx = cid == 0 ? slot0 : (pair_of ? (int64_t)pair_of[lin] : lin);
            if (idx < 0) continue;
            float4 bb = cid == 0 ? bb0 : aabb[idx];
            if (bb.z <= bb.x || bb.w <= bb.y) continue;
            any_view = true;
            CamDev cam = load_cam(viewmats, intrins, cid);
            float4* vr = (float4*)(v_screen + idx);
            float4 va, vb, vc4;
            if (cid == 0) { va = vr0[0]; vb = vr0[1]; vc4 = vr0[2]; }
            else { va = vr[0]; vb = vr[1]; vc4 = vr[2]; }
            if (clear_v_screen) {   // leave the record ready for the next view's reductions
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                vr[0] = zero; vr[1] = zero; vr[2] = zero;
            }
            ProjGeom g;
            LensDist lens = {};
            if (DIST) lens = load_lens(da, cid);
            project_geom<MODEL, DIST, true>(cam, lens, W, antialiased != 0, mean, quat, scale, in_op, g);
            // ---- conic -> blurred 2D covariance
            float v0 = vb.x, v1 = vb.y, v2 = vb.z;
            float invdet = 1.0f / g.det;
            float vD = -(v0 * g.conic[0] + v1 * g.conic[1] + v2 * g.conic[2]) * invdet;
            float G00 = v2 * invdet + vD * g.c11;
            float G11 = v0 * invdet + vD * g.c00;
            float G01 = 0.5f * (-v1 * invdet - 2.f * vD * g.c01);
            float v_opac = vb.w;
            if (antialiased) {
                // opacity *= sqrt(max(0, det_orig / det_blur))
                const float eps2d = 0.1f;
                float o00 = g.c00 - eps2d, o11 = g.c11 - eps2d;
                float det_orig = o00 * o11 - g.c01 * g.c01;
                float ratio = det_orig * invdet;
                if (ratio > 0.f) {
                    float comp = sqrtf(ratio);
                    float op0 = g.opacity / comp;          // pre-compensation opacity
                    float v_comp = v_opac * op0;
                    float v_ratio = v_comp * 0.5f / comp;
                    float v_do = v_ratio * invdet, v_db = -v_ratio * ratio * invdet;
                    G00 += v_do * o11 + v_db * g.c11;
                    G11 += v_do * o00 + v_db * g.c00;
                    G01 += 0.5f * (-2.f * g.c01 * (v_do + v_db));
                    v_opac *= comp;
                    g.opacity = op0;
                } else {
                    v_opac = 0.f;
                }
            }
            // ---- cov2d = J covc J^T : v_J = 2 G J covc, v_covc = J^T G J
            const float* c = g.covc;
            float x = g.mc[0], y = g.mc[1], z = g.mc[2];
            float vmc[3] = {0.f, 0.f, 0.f};
            float vC[9];
            if (MODEL == SSB_CAMERA_PINHOLE && !DIST) {
                float JC0[3] = {g.J00 * c[0] + g.J02 * c[2], g.J00 * c[1] + g.J02 * c[4], g.J00 * c[2] + g.J02 * c[5]};
                float JC1[3] = {g.J11 * c[1] + g.J12 * c[2], g.J11 * c[3] + g.J12 * c[4], g.J11 * c[4] + g.J12 * c[5]};
                float vJ00 = 2.f * (G00 * JC0[0] + G01 * JC1[0]);
                float vJ02 = 2.f * (G00 * JC0[2] + G01 * JC1[2]);
                float vJ11 = 2.f * (G01 * JC0[1] + G11 * JC1[1]);
                float vJ12 = 2.f * (G01 * JC0[2] + G11 * JC1[2]);
                // J rows: r0 = (J00, 0, J02), r1 = (0, J11, J12); v_covc[i][j] = sum_ab J[a][i] G[a][b] J[b][j]
                float r0[3] = {g.J00, 0.f, g.J02}, r1[3] = {0.f, g.J11, g.J12};
#pragma unroll
                for (int i = 0; i < 3; ++i)
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        vC[3 * i + j] = r0[i] * (G00 * r0[j] + G01 * r1[j]) + r1[i] * (G01 * r0[j] + G11 * r1[j]);
                // ---- camera-space mean
                float rz = 1.0f / z, rz2 = rz * rz;
                vmc[2] += -cam.fx * rz2 * vJ00 - cam.fy * rz2 * vJ11;
                float width = (float)W;
                float lim_pos = width + 0.3f * (0.5f * width), lim_neg = 0.3f * (0.5f * width);
                if (g.clampx == 0) { vmc[0] += -cam.fx * rz2 * vJ02; vmc[2] += 2.f * cam.fx * x * rz2 * rz * vJ02; }
                else if (g.clampx < 0) vmc[2] += (lim_pos - cam.cx) * rz2 * vJ02;
                else vmc[2] += -(lim_neg + cam.cx) * rz2 * vJ02;
                if (g.clampy == 0) { vmc[1] += -cam.fy * rz2 * vJ12; vmc[2] += 2.f * cam.fy * y * rz2 * rz * vJ12; }
                else if (g.clampy < 0) vmc[2] += (lim_pos - cam.cy) * rz2 * vJ12;
                else vmc[2] += -(lim_neg + cam.cy) * rz2 * vJ12;
                vmc[0] += cam.fx * rz * va.x;
                vmc[1] += cam.fy * rz * va.y;
                vmc[2] += -(cam.fx * x * va.x + cam.fy * y * va.y) * rz2;
            } else {
                const float* J = g.Jw;
                float JC0[3] = {J[0] * c[0] + J[1] * c[1] + J[2] * c[2], J[0] * c[1] + J[1] * c[3] + J[2] * c[4], J[0] * c[2] + J[1] * c[4] + J[2] * c[5]};
                float JC1[3] = {J[3] * c[0] + J[4] * c[1] + J[5] * c[2], J[3] * c[1] + J[4] * c[3] + J[5] * c[4], J[3] * c[2] + J[4] * c[4] + J[5] * c[5]};
                float vJ[6];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    vJ[j] = 2.f * (G00 * JC0[j] + G01 * JC1[j]);
                    vJ[3 + j] = 2.f * (G01 * JC0[j] + G11 * JC1[j]);
                }
#pragma unroll
                for (int i = 0; i < 3; ++i)
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        vC[3 * i + j] = J[i] * (G00 * J[j] + G01 * J[3 + j]) + J[3 + i] * (G01 * J[j] + G11 * J[3 + j]);
                // ---- camera-space mean: v_mc = J^T v_mean2d + sum_ij vJ[i][j] dJ[i][j]/d mc
                D3 pd[3] = {{x, 1.f, 0.f, 0.f}, {y, 0.f, 1.f, 0.f}, {z, 0.f, 0.f, 1.f}};
                D3 uvd[2], Jd[6];
                if (DIST) { D3 nd[2]; project_mean_dist<MODEL, D3>(pd, cam, lens, W, uvd, Jd, nd); }
                else project_mean_wide<MODEL, D3>(pd, cam.fx, cam.fy, cam.cx, cam.cy, uvd, Jd);
#pragma unroll
                for (int e = 0; e < 6; ++e) { vmc[0] += vJ[e] * Jd[e].dx; vmc[1] += vJ[e] * Jd[e].dy; vmc[2] += vJ[e] * Jd[e].dz; }
                if (DIST) {     // the pinhole's limited third column is not d(uv)/dz: take the derivatives of uv themselves
                    vmc[0] += uvd[0].dx * va.x + uvd[1].dx * va.y;
                    vmc[1] += uvd[0].dy * va.x + uvd[1].dy * va.y;
                    vmc[2] += uvd[0].dz * va.x + uvd[1].dz * va.y;
                } else {
                    vmc[0] += J[0] * va.x + J[3] * va.y;
                    vmc[1] += J[1] * va.x + J[4] * va.y;
                    vmc[2] += J[2] * va.x + J[5] * va.y;
                }
            }
            float vdl = vc4.w / g.len;   // depth = |mc|
            vmc[0] += vdl * x; vmc[1] += vdl * y; vmc[2] += vdl * z;
            const float* R = cam.R;
#pragma unroll
            for (int j = 0; j < 3; ++j) g_mean[j] += finite_or_zero(R[j] * vmc[0] + R[3 + j] * vmc[1] + R[6 + j] * vmc[2]);
            // ---- covc = Wm diag(s^2) Wm^T, Wm = R Rq
            // v_Wm = 2 vC Wm diag(s^2);  v_s2[j] = sum_{ik} Wm[i][j] vC[i][k] Wm[k][j]
            const float* Wm = g.W;
            float s2[3] = {g.s[0] * g.s[0], g.s[1] * g.s[1], g.s[2] * g.s[2]};
            float vCW[9];
#pragma unroll
            for (int i = 0; i < 3; ++i)
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    vCW[3 * i + j] = vC[3 * i] * Wm[j] + vC[3 * i + 1] * Wm[3 + j] + vC[3 * i + 2] * Wm[6 + j];
            float vscale[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                float vs2 = Wm[j] * vCW[j] + Wm[3 + j] * vCW[3 + j] + Wm[6 + j] * vCW[6 + j];
                vscale[j] = vs2 * 2.f * s2[j];   // d s^2 / d log s = 2 s^2
                g_scale[j] += finite_or_zero(vscale[j]);
            }
            // v_Rq = R^T v_Wm, v_Wm[i][j] = 2 vCW[i][j] s2[j]
            float vRq[9];
#pragma unroll
            for (int i = 0; i < 3; ++i)
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    vRq[3 * i + j] = 2.f * s2[j] * (R[i] * vCW[j] + R[3 + i] * vCW[3 + j] + R[6 + i] * vCW[6 + j]);
            float qw = g.qn[0], qx = g.qn[1], qy = g.qn[2], qz = g.qn[3];
            float vq[4];
            vq[0] = 2.f * (-qz * vRq[1] + qy * vRq[2] + qz * vRq[3] - qx * vRq[5] - qy * vRq[6] + qx * vRq[7]);
            vq[1] = 2.f * (qy * vRq[1] + qz * vRq[2] + qy * vRq[3] - 2.f * qx * vRq[4] - qw * vRq[5] + qz * vRq[6] + qw * vRq[7] - 2.f * qx * vRq[8]);
            vq[2] = 2.f * (-2.f * qy * vRq[0] + qx * vRq[1] + qw * vRq[2] + qx * vRq[3] + qz * vRq[5] - qw * vRq[6] + qz * vRq[7] - 2.f * qy * vRq[8]);
            vq[3] = 2.f * (-2.f * qz * vRq[0] - qw * vRq[1] + qx * vRq[2] + qw * vRq[3] - 2.f * qz * vRq[4] + qy * vRq[5] + qx * vRq[6] + qy * vRq[7]);
            float dq = qw * vq[0] + qx * vq[1] + qy * vq[2] + qz * vq[3];
#pragma unroll
            for (int i = 0; i < 4; ++i) g_quat[i] += finite_or_zero((vq[i] - g.qn[i] * dq) * g.qinv);
            g_op += finite_or_zero(v_opac * g.opacity * (1.0f - g.opacity));
            // ---- SH
            float d[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) d[j] = mean[j] + (R[j] * cam.t[0] + R[3 + j] * cam.t[1] + R[6 + j] * cam.t[2]);
            float inv = rsqrtf(d[0] * d[0] + d[1] * d[1] + d[2] * d[2]);
            float nx = d[0] * inv, ny = d[1] * inv, nz = d[2] * inv;
            float b[kNumSh];
            sh_basis(nx, ny, nz, b);
            float vcol[3] = {vc4.x, vc4.y, vc4.z};
#pragma unroll
            for (int ch = 0; ch < 3; ++ch) {
                float raw = kShC0 * dc_in[ch];
#pragma unroll
                for (int j = 0; j < kNumSh; ++j) if (j < da.n_sh) raw += b[j] * sh[3 * j + ch];
                if (!(raw >= -0.5f)) vcol[ch] = 0.f;
                vcol[ch] = finite_or_zero(vcol[ch]);
                g_dc[ch] += kShC0 * vcol[ch];
            }
            float w[kNumSh];
#pragma unroll
            for (int j = 0; j < kNumSh; ++j) {
                const bool on = j < da.n_sh;       // a band above the active degree takes no gradient and moves no direction
                w[j] = on ? sh[3 * j] * vcol[0] + sh[3 * j + 1] * vcol[1] + sh[3 * j + 2] * vcol[2] : 0.f;
                const float bj = on ? b[j] : 0.f;
                if (MULTI_VIEW) { shg[3 * j] += bj * vcol[0]; shg[3 * j + 1] += bj * vcol[1]; shg[3 * j + 2] += bj * vcol[2]; }
                else { shg[3 * j] = bj * vcol[0]; shg[3 * j + 1] = bj * vcol[1]; shg[3 * j + 2] = bj * vcol[2]; }
            }
            float vn[3];
            sh_basis_vjp(nx, ny, nz, w, vn);
            float dn = nx * vn[0] + ny * vn[1] + nz * vn[2];
            g_mean[0] += finite_or_zero((vn[0] - nx * dn) * inv);
            g_mean[1] += finite_or_zero((vn[1] - ny * dn) * inv);
            g_mean[2] += finite_or_zero((vn[2] - nz * dn) * inv);
        }
        if (!MULTI_VIEW && !any_view) {
            // culled in the only view: the span still holds SH values, not gradients
            float* shg0 = shg_s + threadIdx.x * kShPerSplat;
#pragma unroll
            for (int j = 0; j < kShPerSplat; ++j) shg0[j] = 0.f;
        }
        if (accumulate) {
            if (any_view) {      // a splat no view sees adds nothing
#pragma unroll
            for (int j = 0; j < 3; ++j) { atomicAdd(&gr.means[3 * gid + j], g_mean[j]); atomicAdd(&gr.scales[3 * gid + j], g_scale[j]); atomicAdd(&gr.features_dc[3 * gid + j], g_dc[j]); }
            red_add_v4(gr.quats + 4 * gid, g_quat[0], g_quat[1], g_quat[2], g_quat[3]);
            atomicAdd(&gr.opacities[gid], g_op);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 3; ++j) { gr.means[3 * gid + j] = g_mean[j]; gr.scales[3 * gid + j] = g_scale[j]; gr.features_dc[3 * gid + j] = g_dc[j]; }
            ((float4*)gr.quats)[gid] = make_float4(g_quat[0], g_quat[1], g_quat[2], g_quat[3]);
            gr.opacities[gid] = g_op;
        }
    }
    __syncthreads();
    float* out = gr.features_sh + first * kShPerSplat;
    if (count == kProjBlock * kShPerSplat && ((uintptr_t)gr.features_sh & 15) == 0) {   // full block of an aligned array
        float4* out4 = (float4*)out;
        const float4* g4 = (const float4*)shg_s;
        if (accumulate) {
            // every address is added to once per launch, so a reduction gives the same sum as
            // load-add-store without waiting for the old value (measured a third faster)
            for (int v = threadIdx.x; v < kProjBlock * kShPerSplat / 4; v += kProjBlock) {
                const float4 g = g4[v];
                if (g.x != 0.f || g.y != 0.f || g.z != 0.f || g.w != 0.f)      // a culled splat's 45 zeros cost no traffic
                    red_add_v4(out + 4 * v, g.x, g.y, g.z, g.w);
            }
        } else {
            for (int v = threadIdx.x; v < kProjBlock * kShPerSplat / 4; v += kProjBlock) out4[v] = g4[v];
        }
    } else if (accumulate) for (int i = threadIdx.x; i < count; i += kProjBlock) out[i] += shg_s[i];
    else for (int i = threadIdx.x; i < count; i += kProjBlock) out[i] = shg_s[i];
}

// ADD: the arrays are accumulated into (gradient records onto running gradient arrays) instead of overwritten.
template <bool ADD>
__global__ void screen_unpack_kernel(const SsbScreenRec* __restrict__ s, int64_t m, float* xy, float* depth, float* conic, float* opac, float* rgb) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const float4* r = (const float4*)(s + i);
    float4 a = r[0], b = r[1], c = r[2];
    auto put = [](float* dst, float v) { if (ADD) *dst += v; else *dst = v; };
    if (xy) { put(xy + 2 * i, a.x); put(xy + 2 * i + 1, a.y); }
    if (depth) put(depth + i, c.w);
    if (conic) { put(conic + 3 * i, b.x); put(conic + 3 * i + 1, b.y); put(conic + 3 * i + 2, b.z); }
    if (opac) put(opac + i, b.w);
    if (rgb) { put(rgb + 3 * i, c.x); put(rgb + 3 * i + 1, c.y); put(rgb + 3 * i + 2, c.z); }
}

__global__ void screen_pack_kernel(const float* xy, const float* depth, const float* conic, const float* opac, const float* rgb, int64_t m, SsbScreenRec* s) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    float ca = conic[3 * i], cb = conic[3 * i + 1], cc = conic[3 * i + 2], op = opac[i];
    // footprint half extents from the conic: cov = conic^-1
    float hx = 0.f, hy = 0.f;
    float det = ca * cc - cb * cb;
    if (op > kAlphaThreshold && det > 0.f) {
        float e = sqrtf(2.0f * logf(op / kAlphaThreshold)) * 1.0005f;
        hx = e * sqrtf(cc / det) + 1e-3f;
        hy = e * sqrtf(ca / det) + 1e-3f;
    }
    float4* r = (float4*)(s + i);
    r[0] = make_float4(xy[2 * i], xy[2 * i + 1], hx, hy);
    r[1] = make_float4(ca, cb, cc, op);
    r[2] = make_float4(rgb[3 * i], rgb[3 * i + 1], rgb[3 * i + 2], depth[i]);
}

// The (camera model, distortion tier) pairs of the reference's instantiation table
// (src/kernels/projection/CameraVariants.cuh:11-22): every tier for the pinhole, OpenCV and thin prism for the two
// fisheyes (no COLMAP fisheye model uses the rational tier), none for the equirectangular camera.
static bool distortion_variant_built(int model, int tier) {
    if (tier == SSB_DISTORTION_NONE) return true;
    if (tier == SSB_DISTORTION_OPENCV || tier == SSB_DISTORTION_THIN_PRISM) return model != SSB_CAMERA_EQUIRECT;
    if (tier == SSB_DISTORTION_RATIONAL) return model == SSB_CAMERA_PINHOLE;
    return false;
}

// SH coefficients past DC that the active degree uses: SsbCameras::sh_degree_plus1 = 0 means all 15 (degree 3)
static int active_sh_count(const SsbCameras* cams) {
    const int p1 = cams->sh_degree_plus1;
    return (p1 >= 1 && p1 <= 4) ? p1 * p1 - 1 : kNumSh;
}

static int check_shq(const SsbSplats* splats, const SsbShQuant* shq, SsbShQuant& out) {
    out = SsbShQuant{nullptr, nullptr, 32, 0, 256};
    if (shq && shq->packed && (shq->bits == 8 || shq->bits == 16)) {
        out = *shq;
        if (out.bounds_stride <= 0) out.bounds_stride = (int64_t)256 * 3 * kNumSh;
        SSB_REQUIRE(out.bounds != nullptr, "quantised SH needs a bounds table");
    } else {
        SSB_REQUIRE(splats->features_sh != nullptr, "features_sh is NULL and no quantised SH was given");
    }
    return SSB_OK;
}

}  // namespace ssb

extern "C" {

int ssb_project_fwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                    float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(splats && cams && d_aabb && d_depths && d_screen, "ssb_project_fwd: NULL argument");
    SSB_REQUIRE(n >= 0 && cams->count >= 0 && cams->width > 0 && cams->height > 0, "ssb_project_fwd: bad sizes");
    if (cams->model != SSB_CAMERA_PINHOLE && cams->model != SSB_CAMERA_FISHEYE && cams->model != SSB_CAMERA_EQUISOLID && cams->model != SSB_CAMERA_EQUIRECT) {
        set_error("ssb_project_fwd: camera model %d not supported", cams->model); return SSB_ERR_UNSUPPORTED;
    }
    if (!distortion_variant_built(cams->model, cams->distortion)) {
        set_error("ssb_project_fwd: unsupported camera model / distortion tier (%d, %d)", cams->model, cams->distortion); return SSB_ERR_UNSUPPORTED;
    }
    SSB_REQUIRE(cams->sh_degree_plus1 >= 0 && cams->sh_degree_plus1 <= 4, "ssb_project_fwd: sh_degree_plus1 must be 0 (all bands) or 1..4");
    const DistArgs da = {cams->d_dist_coeffs, cams->distortion, active_sh_count(cams)};
    SSB_REQUIRE((int64_t)cams->count * n < ((int64_t)1 << 31), "ssb_project_fwd: views * splats must fit int32 flatten ids");
    SsbShQuant q;
    int e = check_shq(splats, shq, q);
    if (e) return e;
    if (n == 0 || cams->count == 0) return SSB_OK;
    dim3 grid((unsigned)ceil_div(n, kProjBlock), (unsigned)cams->count);
#define SSB_FWD(MODEL, DIST) project_fwd_kernel<MODEL, 0, DIST><<<grid, kProjBlock, 0, (cudaStream_t)stream>>>( \
        *splats, q, n, cams->d_viewmats, cams->d_intrins, cams->width, cams->height, cams->antialiased, \
        (float4*)d_aabb, d_depths, d_radii, d_screen, PackArgs{}, da)
    const bool dist = cams->distortion != SSB_DISTORTION_NONE;
    if (cams->model == SSB_CAMERA_PINHOLE) { if (dist) SSB_FWD(SSB_CAMERA_PINHOLE, true); else SSB_FWD(SSB_CAMERA_PINHOLE, false); }
    else if (cams->model == SSB_CAMERA_FISHEYE) { if (dist) SSB_FWD(SSB_CAMERA_FISHEYE, true); else SSB_FWD(SSB_CAMERA_FISHEYE, false); }
    else if (cams->model == SSB_CAMERA_EQUISOLID) { if (dist) SSB_FWD(SSB_CAMERA_EQUISOLID, true); else SSB_FWD(SSB_CAMERA_EQUISOLID, false); }
    else SSB_FWD(SSB_CAMERA_EQUIRECT, false);
#undef SSB_FWD
    SSB_LAUNCHED("project_fwd_kernel");
    return SSB_OK;
}

int ssb_project_bwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                    const SsbScreenRec* d_v_screen, const SsbSplats* grads, int accumulate, void* stream) {
    return ssb::launch_project_bwd(splats, shq, n, cams, d_aabb, const_cast<SsbScreenRec*>(d_v_screen), grads, accumulate, 0, stream, nullptr, 0, -1);
}

}  // extern "C"

namespace ssb {

// pass = 1: flags only; pass = 2: compacting pass (flags hold the exclusive scan).
int launch_project_fwd_pack_pass(int pass, const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams,
                                 int32_t* d_flags, float* d_aabb, float* d_depths, float* d_radii, SsbScreenRec* d_screen,
                                 int32_t* d_camera_ids, int32_t* d_gaussian_ids, int64_t capacity, void* stream) {
    if (cams->model != SSB_CAMERA_PINHOLE && cams->model != SSB_CAMERA_FISHEYE && cams->model != SSB_CAMERA_EQUISOLID && cams->model != SSB_CAMERA_EQUIRECT) {
        set_error("ssb_project_fwd_packed: camera model %d not supported", cams->model); return SSB_ERR_UNSUPPORTED;
    }
    if (!distortion_variant_built(cams->model, cams->distortion)) {
        set_error("ssb_project_fwd_packed: unsupported camera model / distortion tier (%d, %d)", cams->model, cams->distortion); return SSB_ERR_UNSUPPORTED;
    }
    SSB_REQUIRE(cams->sh_degree_plus1 >= 0 && cams->sh_degree_plus1 <= 4, "ssb_project_fwd_packed: sh_degree_plus1 must be 0 (all bands) or 1..4");
    const DistArgs da = {cams->d_dist_coeffs, cams->distortion, active_sh_count(cams)};
    const bool dist = cams->distortion != SSB_DISTORTION_NONE;
    SSB_REQUIRE((int64_t)cams->count * n < ((int64_t)1 << 31), "ssb_project_fwd_packed: views * splats must fit int32");
    SsbShQuant q;
    int e = check_shq(splats, shq, q);
    if (e) return e;
    if (n == 0 || cams->count == 0) return SSB_OK;
    dim3 grid((unsigned)ceil_div(n, kProjBlock), (unsigned)cams->count);
    const PackArgs pk = {d_flags, d_camera_ids, d_gaussian_ids, capacity};
#define SSB_FWDP(MODEL, PASS, DIST) project_fwd_kernel<MODEL, PASS, DIST><<<grid, kProjBlock, 0, (cudaStream_t)stream>>>( \
        *splats, q, n, cams->d_viewmats, cams->d_intrins, cams->width, cams->height, cams->antialiased, \
        (float4*)d_aabb, d_depths, d_radii, d_screen, pk, da)
#define SSB_FWDP_MODEL(PASS) \
    do { \
        if (cams->model == SSB_CAMERA_PINHOLE) { if (dist) SSB_FWDP(SSB_CAMERA_PINHOLE, PASS, true); else SSB_FWDP(SSB_CAMERA_PINHOLE, PASS, false); } \
        else if (cams->model == SSB_CAMERA_FISHEYE) { if (dist) SSB_FWDP(SSB_CAMERA_FISHEYE, PASS, true); else SSB_FWDP(SSB_CAMERA_FISHEYE, PASS, false); } \
        else if (cams->model == SSB_CAMERA_EQUISOLID) { if (dist) SSB_FWDP(SSB_CAMERA_EQUISOLID, PASS, true); else SSB_FWDP(SSB_CAMERA_EQUISOLID, PASS, false); } \
        else SSB_FWDP(SSB_CAMERA_EQUIRECT, PASS, false); \
    } while (0)
    if (pass == 1) SSB_FWDP_MODEL(1); else SSB_FWDP_MODEL(2);
#undef SSB_FWDP_MODEL
#undef SSB_FWDP
    SSB_LAUNCHED("project_fwd_kernel<packed>");
    return SSB_OK;
}

int launch_project_bwd(const SsbSplats* splats, const SsbShQuant* shq, int64_t n, const SsbCameras* cams, const float* d_aabb,
                       SsbScreenRec* d_v_screen, const SsbSplats* grads, int accumulate, int clear_v_screen, void* stream,
                       const int32_t* d_pair_of, int64_t range_first, int64_t range_count) {
    SSB_REQUIRE(splats && cams && d_aabb && d_v_screen && grads, "ssb_project_bwd: NULL argument");
    SSB_REQUIRE(grads->means && grads->quats && grads->scales && grads->opacities && grads->features_dc && grads->features_sh,
                "ssb_project_bwd: every gradient array must be given");
    if (cams->model != SSB_CAMERA_PINHOLE && cams->model != SSB_CAMERA_FISHEYE && cams->model != SSB_CAMERA_EQUISOLID && cams->model != SSB_CAMERA_EQUIRECT) {
        set_error("ssb_project_bwd: camera model %d not supported", cams->model); return SSB_ERR_UNSUPPORTED;
    }
    if (!distortion_variant_built(cams->model, cams->distortion)) {
        set_error("ssb_project_bwd: unsupported camera model / distortion tier (%d, %d)", cams->model, cams->distortion); return SSB_ERR_UNSUPPORTED;
    }
    SSB_REQUIRE(cams->sh_degree_plus1 >= 0 && cams->sh_degree_plus1 <= 4, "ssb_project_bwd: sh_degree_plus1 must be 0 (all bands) or 1..4");
    const DistArgs da = {cams->d_dist_coeffs, cams->distortion, active_sh_count(cams)};
    const bool dist = cams->distortion != SSB_DISTORTION_NONE;
    SsbShQuant q;
    int e = check_shq(splats, shq, q);
    if (e) return e;
    if (range_count < 0) { range_first = 0; range_count = n; }     // the whole array
    SSB_REQUIRE(range_first >= 0 && range_first + range_count <= n && range_first % kProjBlock == 0, "ssb_project_bwd: bad splat range");
    if (range_count == 0) return SSB_OK;
    const int64_t range_end = range_first + range_count;
#define SSB_BWD(MULTI, MODEL, DIST) project_bwd_kernel<MULTI, MODEL, DIST><<<(unsigned)ceil_div(range_count, kProjBlock), kProjBlock, 0, (cudaStream_t)stream>>>( \
        *splats, q, n, cams->count, cams->d_viewmats, cams->d_intrins, cams->width, cams->height, cams->antialiased, \
        (const float4*)d_aabb, d_v_screen, *grads, accumulate, clear_v_screen, d_pair_of, range_first, range_end, da)
#define SSB_BWD_MODEL(MODEL) \
    do { \
        if (dist) { if (multi) SSB_BWD(true, MODEL, true); else SSB_BWD(false, MODEL, true); } \
        else { if (multi) SSB_BWD(true, MODEL, false); else SSB_BWD(false, MODEL, false); } \
    } while (0)
    const bool multi = cams->count != 1;
    if (cams->model == SSB_CAMERA_PINHOLE) SSB_BWD_MODEL(SSB_CAMERA_PINHOLE);
    else if (cams->model == SSB_CAMERA_FISHEYE) SSB_BWD_MODEL(SSB_CAMERA_FISHEYE);
    else if (cams->model == SSB_CAMERA_EQUISOLID) SSB_BWD_MODEL(SSB_CAMERA_EQUISOLID);
    else { if (multi) SSB_BWD(true, SSB_CAMERA_EQUIRECT, false); else SSB_BWD(false, SSB_CAMERA_EQUIRECT, false); }
#undef SSB_BWD_MODEL
#undef SSB_BWD
    SSB_LAUNCHED("project_bwd_kernel");
    return SSB_OK;
}

}  // namespace ssb

extern "C" {

int ssb_screen_unpack(const SsbScreenRec* d_screen, int64_t m, float* d_xy, float* d_depth, float* d_conic, float* d_opac, float* d_rgb, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_screen && m >= 0, "ssb_screen_unpack: bad argument");
    if (m == 0) return SSB_OK;
    screen_unpack_kernel<false><<<(unsigned)ceil_div(m, 256), 256, 0, (cudaStream_t)stream>>>(d_screen, m, d_xy, d_depth, d_conic, d_opac, d_rgb);
    SSB_LAUNCHED("screen_unpack_kernel");
    return SSB_OK;
}

int ssb_screen_unpack_add(const SsbScreenRec* d_records, int64_t m, float* d_xy, float* d_depth, float* d_conic, float* d_opac, float* d_rgb, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_records && m >= 0, "ssb_screen_unpack_add: bad argument");
    if (m == 0) return SSB_OK;
    screen_unpack_kernel<true><<<(unsigned)ceil_div(m, 256), 256, 0, (cudaStream_t)stream>>>(d_records, m, d_xy, d_depth, d_conic, d_opac, d_rgb);
    SSB_LAUNCHED("screen_unpack_kernel");
    return SSB_OK;
}

int ssb_screen_pack(const float* d_xy, const float* d_depth, const float* d_conic, const float* d_opac, const float* d_rgb, int64_t m,
                    SsbScreenRec* d_screen, void* stream) {
    using namespace ssb;
    SSB_REQUIRE(d_xy && d_depth && d_conic && d_opac && d_rgb && d_screen && m >= 0, "ssb_screen_pack: bad argument");
    if (m == 0) return SSB_OK;
    screen_pack_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, (cudaStream_t)stream>>>(d_xy, d_depth, d_conic, d_opac, d_rgb, m, d_screen);
    SSB_LAUNCHED("screen_pack_kernel");
    return SSB_OK;
}

}  // extern "C"
