// adop_math.h — the arithmetic specification of the one-pixel point rasterizer.
//
// Every function here compiles both for the host (g++) and for the device (nvcc) and is written so that
// both produce the same bits: a fixed operation order, fused multiply-adds only where fmaf() is written out
// (correctly rounded on both sides), no fast-math, IEEE division and square root, own polynomial
// atan/atan2/acos instead of the two different libm versions.
// Build rules that the bit-equality relies on:  g++ -ffp-contract=off (-mfma makes fmaf one instruction)
// and nvcc -fmad=false (-prec-div=true and -prec-sqrt=true are nvcc defaults).
// The point kernels are instruction-issue bound as much as memory bound, so the forward projection is
// written for a short instruction stream: Horner forms in fmaf, one reciprocal instead of several divisions.
//
// The reference (darglein/ADOP) takes all of this arithmetic from the saiga library, whose source is not
// part of the reference tree; each function states the reference call site whose contract it restates and
// marks the choices that had to be made where that contract is silent.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define ADOP_HD __host__ __device__ __forceinline__
#else
#define ADOP_HD inline
#endif

namespace adop {

constexpr int kMaxLayers    = 8;    // the reference stops at 5 (PointRenderer.h:20)
constexpr int kMaxChannels  = 32;   // the reference's background-gradient kernel stops at 20 (PointRenderer.cu:865)
constexpr int kMaxOcamPoly  = 16;
constexpr float kDepthInit  = 100000.f;  // PointRenderer.cu:1045
constexpr float kDistReject = 100000.f;  // sentinel of PointRendererHelper.h:74

enum CameraModel : int { kPinholeDistortion = 0, kOcam = 1 };  // SceneData.h:27-31

// ---------------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------------
ADOP_HD int float_as_int_bits(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_int(f);
#else
    union { float f; int i; } u; u.f = f; return u.i;
#endif
}

// Round to nearest, ties to even, like __float2int_rn (PointRenderer.cu:266). The clamp makes the
// conversion defined for huge and NaN inputs on both sides: they land far outside every image.
ADOP_HD int round_half_even(float x)
{
    x = fminf(fmaxf(x, -1.0e9f), 1.0e9f);
#if defined(__CUDA_ARCH__)
    return __float2int_rn(x);
#else
    return (int)lrintf(x);  // default rounding mode = to nearest even
#endif
}
// the same for |x| < 1e9 (what project_for_raster guarantees for image positions): no clamp needed
ADOP_HD int round_half_even_bounded(float x)
{
#if defined(__CUDA_ARCH__)
    return __float2int_rn(x);
#else
    return (int)lrintf(x);  // default rounding mode = to nearest even
#endif
}

// 1 / x, correctly rounded on both sides (so the same bits): the device has it as one intrinsic, which is shorter
// than the general division
ADOP_HD float reciprocal(float x)
{
#if defined(__CUDA_ARCH__)
    return __frcp_rn(x);
#else
    return 1.0f / x;
#endif
}

// Counter-based hash for the per-(view,point) Bernoulli drop-out decision. The reference draws
// bernoulli_() into a [B,N] float tensor (PointRenderer.cu:1081-1088); a hash needs no memory.
ADOP_HD uint32_t hash_u32(uint32_t seed, uint32_t view, uint32_t point)
{
    uint32_t h = seed * 0x9E3779B1u + view * 0x85EBCA77u + 0x165667B1u;
    h ^= point + 0x7F4A7C15u + (h << 6) + (h >> 2);
    h ^= h >> 16; h *= 0x7FEB352Du;
    h ^= h >> 15; h *= 0x846CA68Bu;
    h ^= h >> 16;
    return h;
}
// true = the point is dropped in this view
ADOP_HD bool dropout_decision(float p, uint32_t seed, uint32_t view, uint32_t point)
{
    if (!(p > 0.f)) return false;
    // compare in 24 bits so the float conversion is exact
    uint32_t h24 = hash_u32(seed, view, point) >> 8;
    float u      = (float)h24 * (1.0f / 16777216.0f);
    return u < p;
}

// ---------------------------------------------------------------------------------------------------
// own atan / atan2 / acos (coefficients: least-squares fit on Chebyshev nodes, tests/golden/fit_atan_poly.py)
// ---------------------------------------------------------------------------------------------------
ADOP_HD float atan_core(float x)  // |x| <= tan(pi/8)
{
    float z = x * x;
    float p = -0.06065608f;
    p = fmaf(p, z, 0.10588396f);
    p = fmaf(p, z, -0.14242722f);
    p = fmaf(p, z, 0.19998422f);
    p = fmaf(p, z, -0.33333313f);
    float x3 = z * x;
    return fmaf(x3, p, x);
}
ADOP_HD float atan_unit(float t)  // 0 <= t <= 1
{
    if (t > 0.41421356f)
    {
        float r = (t - 1.0f) / (t + 1.0f);
        return 0.78539816f + atan_core(r);
    }
    return atan_core(t);
}
ADOP_HD float atan_f(float t)
{
    float a = fabsf(t);
    float r;
    if (a > 1.0f) r = 1.57079633f - atan_unit(1.0f / a);
    else          r = atan_unit(a);
    return t < 0.f ? -r : r;
}
ADOP_HD float atan2_f(float y, float x)
{
    float ax = fabsf(x), ay = fabsf(y);
    float r;
    if (ax >= ay) r = (ax == 0.f) ? 0.f : atan_unit(ay / ax);
    else          r = 1.57079633f - atan_unit(ax / ay);
    if (x < 0.f) r = 3.14159265f - r;
    return y < 0.f ? -r : r;
}
ADOP_HD float acos_f(float c)
{
    c = fminf(fmaxf(c, -1.0f), 1.0f);
    float s = sqrtf((1.0f - c) * (1.0f + c));
    return atan2_f(s, c);
}

// ---------------------------------------------------------------------------------------------------
// rigid transform. A pose is the 8-double record of NeuralStructure.cpp:13-27 (a Sophus::SE3d memory
// image): unit quaternion x y z w, translation x y z, one padding double; stored world -> camera.
// The reference casts it to float and rotates with the quaternion (PointRenderer.cu:73). Here the rotation
// matrix is formed once per view in double, rounded to float, and a point costs nine fused multiply-adds:
// the same map, with rounding differences in the last bits only.
// ---------------------------------------------------------------------------------------------------
struct Rigid32 { float r[9]; float t[3]; };  // row-major rotation, translation

ADOP_HD Rigid32 load_rigid(const double* p8)
{
    const double x = p8[0], y = p8[1], z = p8[2], w = p8[3];
    Rigid32 T;
    T.r[0] = (float)(1.0 - 2.0 * (y * y + z * z)); T.r[1] = (float)(2.0 * (x * y - z * w)); T.r[2] = (float)(2.0 * (x * z + y * w));
    T.r[3] = (float)(2.0 * (x * y + z * w)); T.r[4] = (float)(1.0 - 2.0 * (x * x + z * z)); T.r[5] = (float)(2.0 * (y * z - x * w));
    T.r[6] = (float)(2.0 * (x * z - y * w)); T.r[7] = (float)(2.0 * (y * z + x * w)); T.r[8] = (float)(1.0 - 2.0 * (x * x + y * y));
    T.t[0] = (float)p8[4]; T.t[1] = (float)p8[5]; T.t[2] = (float)p8[6];
    return T;
}

struct V3 { float x, y, z; };
struct V2 { float x, y; };

ADOP_HD V3 rotate(const Rigid32& T, V3 v)
{
    V3 o;
    o.x = fmaf(T.r[0], v.x, fmaf(T.r[1], v.y, T.r[2] * v.z));
    o.y = fmaf(T.r[3], v.x, fmaf(T.r[4], v.y, T.r[5] * v.z));
    o.z = fmaf(T.r[6], v.x, fmaf(T.r[7], v.y, T.r[8] * v.z));
    return o;
}
ADOP_HD V3 rotate_inv(const Rigid32& T, V3 v)
{
    V3 o;
    o.x = fmaf(T.r[0], v.x, fmaf(T.r[3], v.y, T.r[6] * v.z));
    o.y = fmaf(T.r[1], v.x, fmaf(T.r[4], v.y, T.r[7] * v.z));
    o.z = fmaf(T.r[2], v.x, fmaf(T.r[5], v.y, T.r[8] * v.z));
    return o;
}
// TransformPoint (PointRendererHelper.h:55): view = R p + t
ADOP_HD V3 transform_point(const Rigid32& T, V3 p)
{
    V3 o;
    o.x = fmaf(T.r[0], p.x, fmaf(T.r[1], p.y, fmaf(T.r[2], p.z, T.t[0])));
    o.y = fmaf(T.r[3], p.x, fmaf(T.r[4], p.y, fmaf(T.r[5], p.z, T.t[1])));
    o.z = fmaf(T.r[6], p.x, fmaf(T.r[7], p.y, fmaf(T.r[8], p.z, T.t[2])));
    return o;
}

// 10-bit-per-axis packed normal (NeuralPointCloudCuda.h:96). The reference's bit layout lives in saiga;
// this layout is this library's own: bits 0-9 x, 10-19 y, 20-29 z, each u/1023*2-1.
ADOP_HD V3 unpack_normal_10bit(int32_t enc)
{
    uint32_t e = (uint32_t)enc;
    V3 n;
    n.x = (float)(e & 1023u) * (2.0f / 1023.0f) - 1.0f;
    n.y = (float)((e >> 10) & 1023u) * (2.0f / 1023.0f) - 1.0f;
    n.z = (float)((e >> 20) & 1023u) * (2.0f / 1023.0f) - 1.0f;
    return n;
}
inline int32_t pack_normal_10bit(float x, float y, float z)
{
    auto q = [](float v) { v = fminf(fmaxf(v, -1.f), 1.f); return (uint32_t)lrintf((v + 1.0f) * 0.5f * 1023.0f); };
    return (int32_t)(q(x) | (q(y) << 10) | (q(z) << 20));
}

// ---------------------------------------------------------------------------------------------------
// pinhole intrinsics: 5 coefficients fx fy cx cy s (SceneData.h:182); the same 5-vector is the crop
// transform of a view (SceneData.h:46).  u = fx x + s y + cx ; v = fy y + cy
// ---------------------------------------------------------------------------------------------------
struct Intr5 { float fx, fy, cx, cy, s; };

ADOP_HD Intr5 load_intr5(const float* p) { Intr5 K; K.fx = p[0]; K.fy = p[1]; K.cx = p[2]; K.cy = p[3]; K.s = p[4]; return K; }
ADOP_HD V2 normalized_to_image(const Intr5& K, V2 p)
{
    V2 o;
    o.x = fmaf(K.fx, p.x, fmaf(K.s, p.y, K.cx));
    o.y = fmaf(K.fy, p.y, K.cy);
    return o;
}
ADOP_HD V2 image_to_normalized(const Intr5& K, V2 ip)  // unproject2 (EnvironmentMap.cu:82)
{
    V2 o;
    o.y = (ip.y - K.cy) / K.fy;
    o.x = ((ip.x - K.cx) - K.s * o.y) / K.fx;
    return o;
}
ADOP_HD Intr5 scale_intr(const Intr5& K, float a)  // IntrinsicsPinholef::scale (PointRenderer.cu:616)
{
    Intr5 o; o.fx = K.fx * a; o.fy = K.fy * a; o.cx = K.cx * a; o.cy = K.cy * a; o.s = K.s * a; return o;
}

// ---------------------------------------------------------------------------------------------------
// 8-coefficient rational distortion, order k1 k2 k3 k4 k5 k6 p1 p2 (PointRenderer.cu:663-673), the
// published OpenCV model. Points whose squared radius exceeds cutoff^2 are rejected (the reference's
// distortNormalizedPoint returns a sentinel there, PointRendererHelper.h:72-77; whether it compares r
// or r^2, > or >=, is this library's choice: r^2 > cutoff^2).
// ---------------------------------------------------------------------------------------------------
struct Dist8 { float k1, k2, k3, k4, k5, k6, p1, p2; };
ADOP_HD Dist8 load_dist8(const float* p)
{
    Dist8 d; d.k1 = p[0]; d.k2 = p[1]; d.k3 = p[2]; d.k4 = p[3]; d.k5 = p[4]; d.k6 = p[5]; d.p1 = p[6]; d.p2 = p[7];
    return d;
}

// J_p (row-major 2x2) and J_d (row-major 2x8) may be null.
ADOP_HD V2 distort(V2 m, const Dist8& d, float cutoff, bool* rejected, float* J_p, float* J_d)
{
    float x = m.x, y = m.y;
    float x2 = x * x, y2 = y * y;
    float r2 = x2 + y2;
    float xy2 = (x + x) * y;
    float num = fmaf(fmaf(fmaf(d.k3, r2, d.k2), r2, d.k1), r2, 1.0f);
    float den = fmaf(fmaf(fmaf(d.k6, r2, d.k5), r2, d.k4), r2, 1.0f);
    float iden = den == 1.0f ? 1.0f : reciprocal(den);  // same bits either way; skips the division for k4 = k5 = k6 = 0
    float rad = num * iden;
    V2 o;
    if (d.p1 == 0.f && d.p2 == 0.f)
    {
        // no tangential part: x * rad + 0 has the same bits as the fused form below
        o.x = x * rad;
        o.y = y * rad;
    }
    else
    {
        float tx = fmaf(d.p1, xy2, d.p2 * fmaf(2.0f, x2, r2));
        float ty = fmaf(d.p2, xy2, d.p1 * fmaf(2.0f, y2, r2));
        o.x = fmaf(x, rad, tx);
        o.y = fmaf(y, rad, ty);
    }
    *rejected = r2 > cutoff * cutoff;
    if (J_p)
    {
        float r4 = r2 * r2;
        float dnum = (d.k1 + 2.0f * d.k2 * r2) + 3.0f * d.k3 * r4;
        float dden = (d.k4 + 2.0f * d.k5 * r2) + 3.0f * d.k6 * r4;
        float drad_dr2 = (dnum * den - num * dden) * (iden * iden);
        float drad_dx = drad_dr2 * (x + x);
        float drad_dy = drad_dr2 * (y + y);
        J_p[0] = ((rad + x * drad_dx) + 2.0f * d.p1 * y) + 6.0f * d.p2 * x;
        J_p[1] = (x * drad_dy + 2.0f * d.p1 * x) + 2.0f * d.p2 * y;
        J_p[2] = (y * drad_dx + 2.0f * d.p1 * x) + 2.0f * d.p2 * y;
        J_p[3] = ((rad + y * drad_dy) + 6.0f * d.p1 * y) + 2.0f * d.p2 * x;
    }
    if (J_d)
    {
        float r4 = r2 * r2;
        float r6 = r4 * r2;
        float a1 = r2 * iden, a2 = r4 * iden, a3 = r6 * iden;
        float nb = -(num * (iden * iden));
        float b1 = nb * r2, b2 = nb * r4, b3 = nb * r6;
        J_d[0] = x * a1; J_d[1] = x * a2; J_d[2] = x * a3; J_d[3] = x * b1; J_d[4] = x * b2; J_d[5] = x * b3;
        J_d[6] = xy2;    J_d[7] = r2 + (x2 + x2);
        J_d[8] = y * a1; J_d[9] = y * a2; J_d[10] = y * a3; J_d[11] = y * b1; J_d[12] = y * b2; J_d[13] = y * b3;
        J_d[14] = r2 + (y2 + y2); J_d[15] = xy2;
    }
    return o;
}

// undistortNormalizedPointSimple (EnvironmentMap.cu:83): plain fixed-point iteration
// m <- (d - tangential(m)) / radial(m); the iteration count (5) is this library's choice.
ADOP_HD V2 undistort_simple(V2 dpt, const Dist8& d)
{
    V2 m = dpt;
    for (int it = 0; it < 5; ++it)
    {
        float x = m.x, y = m.y;
        float x2 = x * x, y2 = y * y;
        float r2 = x2 + y2;
        float xy2 = (x + x) * y;
        float num = fmaf(fmaf(fmaf(d.k3, r2, d.k2), r2, d.k1), r2, 1.0f);
        float den = fmaf(fmaf(fmaf(d.k6, r2, d.k5), r2, d.k4), r2, 1.0f);
        float irad = den / num;
        float tx = fmaf(d.p1, xy2, d.p2 * fmaf(2.0f, x2, r2));
        float ty = fmaf(d.p2, xy2, d.p1 * fmaf(2.0f, y2, r2));
        m.x = (dpt.x - tx) * irad;
        m.y = (dpt.y - ty) * irad;
    }
    return m;
}

// ---------------------------------------------------------------------------------------------------
// projection of one point into one view
// ---------------------------------------------------------------------------------------------------
struct Projected
{
    V2 ip;      // image position before the crop transform
    float z;    // depth; 0 = rejected
    V3 view;    // camera-space position
};

// distort() for the common calibration with only k1 and k2: the same bits as the general form (a zero k3 leaves
// fmaf(k3, r2, k2) = k2, the denominator is exactly 1 and the tangential part is exactly 0) with six fewer
// coefficients to fetch per point.
ADOP_HD V2 distort_radial2(V2 m, float k1, float k2, float cutoff, bool* rejected)
{
    float x = m.x, y = m.y;
    float x2 = x * x, y2 = y * y;
    float r2 = x2 + y2;
    float rad = fmaf(fmaf(k2, r2, k1), r2, 1.0f);
    V2 o;
    o.x = x * rad;
    o.y = y * rad;
    *rejected = r2 > cutoff * cutoff;
    return o;
}

// ProjectPointPinhole (PointRendererHelper.h:49-82) up to the distorted normalised point; the caller applies K.
ADOP_HD Projected project_pinhole_normalized(V3 p, V3 n, bool has_normal, const Rigid32& V, const Dist8& dist,
                                             bool check_normal, float dist_cutoff, bool radial2 = false)
{
    Projected r;
    r.view = transform_point(V, p);
    float z = fmaxf(r.view.z, 0.f);
    r.z = 0.f;
    r.ip.x = 0.f; r.ip.y = 0.f;
    if (!(z > 0.f)) return r;  // behind the camera: the reference carries z = 0 to its skip at PointRenderer.cu:254
    if (check_normal && has_normal)
    {
        V3 vn = rotate(V, n);
        float dt = fmaf(r.view.z, vn.z, fmaf(r.view.y, vn.y, r.view.x * vn.x));
        if (dt > 0.f) return r;
    }
    // DivideByZ (PointRendererHelper.h:70) as one reciprocal and two products
    float iz = reciprocal(r.view.z);
    V2 m;
    m.x = r.view.x * iz;
    m.y = r.view.y * iz;
    bool rejected;
    r.ip = radial2 ? distort_radial2(m, dist.k1, dist.k2, dist_cutoff, &rejected)
                   : distort(m, dist, dist_cutoff, &rejected, nullptr, nullptr);
    r.z = rejected ? 0.f : z;
    return r;
}
ADOP_HD Projected project_pinhole(V3 p, V3 n, bool has_normal, const Rigid32& V, const Intr5& K, const Dist8& dist,
                                  bool check_normal, float dist_cutoff)
{
    Projected r = project_pinhole_normalized(p, n, has_normal, V, dist, check_normal, dist_cutoff);
    r.ip = normalized_to_image(K, r.ip);
    return r;
}

// Omnidirectional (Scaramuzza) model, world->camera polynomial form (PointRendererHelper.h:85-106).
// The reference's ProjectOCam is saiga code; this is the published model with these conventions (own
// choices): camera looks along +z; t = -z/l with l = |(x,y)|; theta = atan(t); rho = sum a_i theta^i;
// (x',y') = (x,y) rho / l ; u = c x' + d y' + cx ; v = e x' + y' + cy ; depth = |p| (SceneData.cpp:694);
// a point is rejected when t > cutoff. Affine parameter order c d e cx cy (SceneData.h:223).
struct Ocam
{
    float c, d, e, cx, cy;
    int npoly;
    float poly[kMaxOcamPoly];
};
ADOP_HD V2 ocam_project(V3 v, const Ocam& o, float cutoff, float* depth, float* J_p /*2x3*/, float* J_aff /*2x5*/)
{
    float l2 = fmaf(v.x, v.x, v.y * v.y);
    float l = fmaxf(sqrtf(l2), 1.0e-12f);
    float il = reciprocal(l);
    float t = -v.z * il;
    if (!J_p && !J_aff && t > cutoff)
    {
        // rejected (see below) and nobody wants the Jacobians: the angle and the polynomial need not be evaluated. On the
        // 100 M point viewer configuration this is more than half of the cloud.
        *depth = 0.f;
        V2 none;
        none.x = none.y = 0.f;
        return none;
    }
    float theta = atan_f(t);
    float rho = 0.f, drho = 0.f;
    for (int i = o.npoly - 1; i >= 0; --i)
    {
        if (J_p) drho = fmaf(drho, theta, rho);
        rho = fmaf(rho, theta, o.poly[i]);
    }
    float s = rho * il;
    float xp = v.x * s, yp = v.y * s;
    V2 ip;
    ip.x = fmaf(o.c, xp, fmaf(o.d, yp, o.cx));
    ip.y = fmaf(o.e, xp, yp + o.cy);
    float nrm = sqrtf(fmaf(v.z, v.z, l2));
    *depth = (t > cutoff) ? 0.f : nrm;
    if (J_p)
    {
        // d theta / d(x,y,z)
        float dth = 1.0f / (1.0f + t * t);
        float il3 = il * il * il;
        float dth_dx = dth * (v.z * v.x * il3);
        float dth_dy = dth * (v.z * v.y * il3);
        float dth_dz = dth * (-il);
        // s = rho / l
        float ds_dx = drho * dth_dx * il - rho * v.x * il3;
        float ds_dy = drho * dth_dy * il - rho * v.y * il3;
        float ds_dz = drho * dth_dz * il;
        float dxp_dx = s + v.x * ds_dx, dxp_dy = v.x * ds_dy, dxp_dz = v.x * ds_dz;
        float dyp_dx = v.y * ds_dx, dyp_dy = s + v.y * ds_dy, dyp_dz = v.y * ds_dz;
        J_p[0] = o.c * dxp_dx + o.d * dyp_dx; J_p[1] = o.c * dxp_dy + o.d * dyp_dy; J_p[2] = o.c * dxp_dz + o.d * dyp_dz;
        J_p[3] = o.e * dxp_dx + dyp_dx;       J_p[4] = o.e * dxp_dy + dyp_dy;       J_p[5] = o.e * dxp_dz + dyp_dz;
    }
    if (J_aff)
    {
        J_aff[0] = xp; J_aff[1] = yp; J_aff[2] = 0.f; J_aff[3] = 1.f; J_aff[4] = 0.f;
        J_aff[5] = 0.f; J_aff[6] = 0.f; J_aff[7] = xp; J_aff[8] = 0.f; J_aff[9] = 1.f;
    }
    return ip;
}

// ProjectPointOcam (PointRendererHelper.h:85-106). Unlike the reference it does not look at the normal
// when the cloud has none (the reference evaluates an uninitialised one there).
ADOP_HD Projected project_ocam(V3 p, V3 n, bool has_normal, const Rigid32& V, const Ocam& o, bool check_normal,
                               float cutoff)
{
    Projected r;
    r.view = transform_point(V, p);
    float z;
    r.ip = ocam_project(r.view, o, cutoff, &z, nullptr, nullptr);
    if (check_normal && has_normal)
    {
        V3 vn = rotate(V, n);
        float dt = fmaf(r.view.z, vn.z, fmaf(r.view.y, vn.y, r.view.x * vn.x));
        if (dt > 0.f) z = 0.f;
    }
    r.z = z;
    return r;
}

// ---------------------------------------------------------------------------------------------------
// One view's camera, gathered from the pose / intrinsics tensors and the ReducedImageInfo, and the
// per-point front end that the three point kernels of the reference share (PointRenderer.cu:227-256,
// 334-359, 413-438): project, reject, apply the crop transform, compute the drop-out radius in pixels.
// ---------------------------------------------------------------------------------------------------
struct ViewCam
{
    Rigid32 V;
    Intr5 crop;
    int model;
    Intr5 K;      // pinhole
    Dist8 dist;   // pinhole
    Ocam ocam;    // omnidirectional
    float w0;     // width of layer 0 (the OCam radius rule uses it as a focal length, PointRenderer.cu:251)
    // pinhole: crop o K as one affine map of the distorted normalised point (formed in double, rounded once):
    // x = a[0] dx + a[1] dy + a[2] ; y = a[3] dy + a[4]. The reference applies K, then the crop (PointRenderer.cu:255).
    float a[5];
    int radial2;  // pinhole with k3 = k4 = k5 = k6 = p1 = p2 = 0: the projection takes distort_radial2
    // The same numbers once more, in the order the radial-only pinhole projection uses them, as five 16-byte vectors
    // (project_for_raster_hot): rows of [R | t], then k1 k2 a0 a1, then a2 a3 a4 and a flag (1.0 = this record may be
    // used: pinhole model, radial-only distortion).
    alignas(16) float hot[20];
};
struct V4 { float x, y, z, w; };

ADOP_HD ViewCam load_view_cam(const double* poses, const float* intrinsics, int intrinsics_cols, int image_index,
                              int camera_index, int camera_model, const float* crop5, int w0)
{
    ViewCam c;
    c.V = load_rigid(poses + (size_t)image_index * 8);
    c.crop = load_intr5(crop5);
    c.model = camera_model;
    c.w0 = (float)w0;
    const float* ip = intrinsics + (size_t)camera_index * intrinsics_cols;
    if (camera_model == kPinholeDistortion)
    {
        c.K = load_intr5(ip);
        c.dist = load_dist8(ip + 5);
        c.radial2 = (c.dist.k3 == 0.f && c.dist.k4 == 0.f && c.dist.k5 == 0.f && c.dist.k6 == 0.f && c.dist.p1 == 0.f &&
                     c.dist.p2 == 0.f) ? 1 : 0;
        c.ocam.npoly = 0;
        const double cfx = crop5[0], cfy = crop5[1], ccx = crop5[2], ccy = crop5[3], cs = crop5[4];
        const double fx = ip[0], fy = ip[1], cx = ip[2], cy = ip[3], sk = ip[4];
        c.a[0] = (float)(cfx * fx);
        c.a[1] = (float)(cfx * sk + cs * fy);
        c.a[2] = (float)(cfx * cx + cs * cy + ccx);
        c.a[3] = (float)(cfy * fy);
        c.a[4] = (float)(cfy * cy + ccy);
    }
    else
    {
        c.ocam.c = ip[0]; c.ocam.d = ip[1]; c.ocam.e = ip[2]; c.ocam.cx = ip[3]; c.ocam.cy = ip[4];
        int m = intrinsics_cols - 5;
        c.ocam.npoly = m < kMaxOcamPoly ? m : kMaxOcamPoly;
        for (int i = 0; i < kMaxOcamPoly; ++i) c.ocam.poly[i] = i < c.ocam.npoly ? ip[5 + i] : 0.f;
        c.K.fx = c.K.fy = 1.f; c.K.cx = c.K.cy = c.K.s = 0.f;
        c.dist.k1 = c.dist.k2 = c.dist.k3 = c.dist.k4 = c.dist.k5 = c.dist.k6 = c.dist.p1 = c.dist.p2 = 0.f;
        c.a[0] = c.a[1] = c.a[2] = c.a[3] = c.a[4] = 0.f;
        c.radial2 = 0;
    }
    for (int r = 0; r < 3; ++r)
    {
        c.hot[4 * r] = c.V.r[3 * r]; c.hot[4 * r + 1] = c.V.r[3 * r + 1]; c.hot[4 * r + 2] = c.V.r[3 * r + 2];
        c.hot[4 * r + 3] = c.V.t[r];
    }
    c.hot[12] = c.dist.k1; c.hot[13] = c.dist.k2; c.hot[14] = c.a[0]; c.hot[15] = c.a[1];
    c.hot[16] = c.a[2]; c.hot[17] = c.a[3]; c.hot[18] = c.a[4];
    c.hot[19] = (camera_model == kPinholeDistortion && c.radial2) ? 1.f : 0.f;
    return c;
}

struct RasterPoint
{
    float x, y;       // position in the (cropped) layer-0 image
    float z;          // depth, > 0
    float radius_px;  // drop-out radius in layer-0 pixels
};

// false = the point does not take part in this view (z == 0 in the reference, PointRenderer.cu:254)
ADOP_HD bool project_for_raster(const ViewCam& c, V3 p, float drop_out_radius, V3 n, bool has_normal,
                                bool check_normal, float dist_cutoff, RasterPoint* out, bool want_radius = true)
{
    Projected pr;
    float focal;
    V2 ip;
    if (c.model == kPinholeDistortion)
    {
        pr = project_pinhole_normalized(p, n, has_normal, c.V, c.dist, check_normal, dist_cutoff, c.radial2 != 0);
        if (!(pr.z > 0.f)) return false;
        focal = c.K.fx * c.crop.fx;
        ip.x = fmaf(c.a[0], pr.ip.x, fmaf(c.a[1], pr.ip.y, c.a[2]));
        ip.y = fmaf(c.a[3], pr.ip.y, c.a[4]);
    }
    else
    {
        pr = project_ocam(p, n, has_normal, c.V, c.ocam, check_normal, dist_cutoff);
        if (!(pr.z > 0.f)) return false;
        focal = c.w0 * c.crop.fx;
        ip = normalized_to_image(c.crop, pr.ip);
    }
    // positions that are not finite or absurdly far off can not land in any layer; rejecting them here keeps the
    // per-layer rounding free of range checks
    if (!(fabsf(ip.x) < 1.0e9f) || !(fabsf(ip.y) < 1.0e9f)) return false;
    out->x = ip.x; out->y = ip.y; out->z = pr.z;
    // only the radius drop-out rule reads it (PointRenderer.cu:261-264); skipping it saves a division
    out->radius_px = want_radius ? focal * drop_out_radius / pr.z : 0.f;
    return true;
}

// project_for_raster for the most common case — pinhole camera with k1, k2 only, no normal test, no radius rule —
// reading the camera from the five vectors of ViewCam::hot (h3.w and h4.* hold k1 k2 a0 a1 | a2 a3 a4 flag). Operation
// for operation the same arithmetic as the general function (transform_point, reciprocal, distort_radial2, the affine
// map, the range check), so the same bits; a CPU test holds the two against each other.
ADOP_HD bool project_for_raster_hot(V4 h0, V4 h1, V4 h2, V4 h3, V4 h4, V3 p, float dist_cutoff, RasterPoint* out)
{
    V3 view;
    view.x = fmaf(h0.x, p.x, fmaf(h0.y, p.y, fmaf(h0.z, p.z, h0.w)));
    view.y = fmaf(h1.x, p.x, fmaf(h1.y, p.y, fmaf(h1.z, p.z, h1.w)));
    view.z = fmaf(h2.x, p.x, fmaf(h2.y, p.y, fmaf(h2.z, p.z, h2.w)));
    float z = fmaxf(view.z, 0.f);
    if (!(z > 0.f)) return false;
    float iz = reciprocal(view.z);
    float x = view.x * iz, y = view.y * iz;
    float x2 = x * x, y2 = y * y;
    float r2 = x2 + y2;
    float rad = fmaf(fmaf(h3.y, r2, h3.x), r2, 1.0f);
    float dx = x * rad, dy = y * rad;
    if (r2 > dist_cutoff * dist_cutoff) return false;
    float ix = fmaf(h3.z, dx, fmaf(h3.w, dy, h4.x));
    float iy = fmaf(h4.y, dy, h4.z);
    if (!(fabsf(ix) < 1.0e9f) || !(fabsf(iy) < 1.0e9f)) return false;
    out->x = ix; out->y = iy; out->z = z;
    out->radius_px = 0.f;
    return true;
}

// ---------------------------------------------------------------------------------------------------
// backward chains (PointRendererHelper.h:109-227). g = gradient w.r.t. the cropped image position.
// TransformPoint's Jacobians: J_point = R ; J_pose = [ I | -[view]x ] for the left update pose <- exp(xi) pose
// (PointRenderer.cu:1653), so g_pose = ( g_v , view x g_v ).
// ---------------------------------------------------------------------------------------------------
struct GradPinhole { float g_point[3]; float g_pose[6]; float g_k[5]; float g_dis[8]; };

ADOP_HD void pose_point_chain(const Rigid32& V, V3 view, V3 gv, float* g_point, float* g_pose)
{
    V3 gp = rotate_inv(V, gv);
    g_point[0] = gp.x; g_point[1] = gp.y; g_point[2] = gp.z;
    g_pose[0] = gv.x; g_pose[1] = gv.y; g_pose[2] = gv.z;
    g_pose[3] = view.y * gv.z - view.z * gv.y;
    g_pose[4] = view.z * gv.x - view.x * gv.z;
    g_pose[5] = view.x * gv.y - view.y * gv.x;
}

ADOP_HD bool project_pinhole_backward(V3 p, V3 n, bool has_normal, V2 g, const Rigid32& V, const Intr5& K,
                                      const Intr5& crop, const Dist8& dist, bool check_normal, float dist_cutoff,
                                      GradPinhole* out)
{
    V3 view = transform_point(V, p);
    if (!(view.z > 0.f)) return false;
    if (check_normal && has_normal)
    {
        V3 vn = rotate(V, n);
        float dt = fmaf(view.z, vn.z, fmaf(view.y, vn.y, view.x * vn.x));
        if (dt > 0.f) return false;
    }
    float iz = reciprocal(view.z);
    V2 m; m.x = view.x * iz; m.y = view.y * iz;
    float Jp[4], Jd[16];
    bool rejected;
    V2 dp = distort(m, dist, dist_cutoff, &rejected, Jp, Jd);
    // crop^T
    float g2x = crop.fx * g.x;
    float g2y = crop.s * g.x + crop.fy * g.y;
    // K: J_k^T
    out->g_k[0] = dp.x * g2x; out->g_k[1] = dp.y * g2y; out->g_k[2] = g2x; out->g_k[3] = g2y; out->g_k[4] = dp.y * g2x;
    // K: J_p^T
    float g1x = K.fx * g2x;
    float g1y = K.s * g2x + K.fy * g2y;
    for (int k = 0; k < 8; ++k) out->g_dis[k] = Jd[k] * g1x + Jd[8 + k] * g1y;
    float gmx = Jp[0] * g1x + Jp[2] * g1y;
    float gmy = Jp[1] * g1x + Jp[3] * g1y;
    // divide by z: J = [[1/z,0,-x/z^2],[0,1/z,-y/z^2]]
    V3 gv;
    gv.x = iz * gmx;
    gv.y = iz * gmy;
    gv.z = -(m.x * iz) * gmx - (m.y * iz) * gmy;
    pose_point_chain(V, view, gv, out->g_point, out->g_pose);
    return true;
}

struct GradOcam { float g_point[3]; float g_pose[6]; float g_affine[5]; };

ADOP_HD bool project_ocam_backward(V3 p, V3 n, bool has_normal, V2 g, const Rigid32& V, const Intr5& crop, const Ocam& o,
                                   bool check_normal, float cutoff, GradOcam* out)
{
    V3 view = transform_point(V, p);
    if (check_normal && has_normal)
    {
        V3 vn = rotate(V, n);
        float dt = fmaf(view.z, vn.z, fmaf(view.y, vn.y, view.x * vn.x));
        if (dt > 0.f) return false;
    }
    float Jp[6], Ja[10], z;
    ocam_project(view, o, cutoff, &z, Jp, Ja);
    float g2x = crop.fx * g.x;
    float g2y = crop.s * g.x + crop.fy * g.y;
    V3 gv;
    gv.x = Jp[0] * g2x + Jp[3] * g2y;
    gv.y = Jp[1] * g2x + Jp[4] * g2y;
    gv.z = Jp[2] * g2x + Jp[5] * g2y;
    for (int k = 0; k < 5; ++k) out->g_affine[k] = Ja[k] * g2x + Ja[5 + k] * g2y;
    pose_point_chain(V, view, gv, out->g_point, out->g_pose);
    return true;
}

// ---------------------------------------------------------------------------------------------------
// environment map lookup coordinate (EnvironmentMap.cu:41-60, 62-105). Returns the sampling position in
// texel units for align_corners / border bilinear interpolation (the grid_sample mode of :143-147).
// The world ray is R^T (m,1) normalised; the reference forms it as V^-1 (m,1) - V^-1 0, the same vector.
// ---------------------------------------------------------------------------------------------------
ADOP_HD V2 spherical_uv(V3 dir)
{
    const float pi = 3.14159265358979323846f;
    float phi = atan2_f(-dir.z, dir.x);
    float x = phi / (2.0f * pi);
    x = x - floorf(x);
    float theta = acos_f(dir.y);
    float y = 1.0f - theta / pi;
    V2 uv; uv.x = x * 2.0f - 1.0f; uv.y = y * 2.0f - 1.0f;
    return uv;
}
ADOP_HD V2 env_uv_for_pixel(int gx, int gy, const Rigid32& V, const Intr5& K, const Dist8& dist, const Intr5& crop_l)
{
    V2 ip; ip.x = (float)gx; ip.y = (float)gy;
    V2 dp = image_to_normalized(K, image_to_normalized(crop_l, ip));
    V2 np = undistort_simple(dp, dist);
    V3 ray; ray.x = np.x; ray.y = np.y; ray.z = 1.0f;
    V3 w = rotate_inv(V, ray);
    float inv = 1.0f / sqrtf((w.x * w.x + w.y * w.y) + w.z * w.z);
    w.x = w.x * inv; w.y = w.y * inv; w.z = w.z * inv;
    return spherical_uv(w);
}
// bilinear taps for uv in [-1,1], align_corners = true, padding = border
struct BilinearTap { int x0, y0, x1, y1; float wx, wy; };
ADOP_HD BilinearTap bilinear_taps(V2 uv, int w, int h)
{
    float fx = (uv.x + 1.0f) * 0.5f * (float)(w - 1);
    float fy = (uv.y + 1.0f) * 0.5f * (float)(h - 1);
    fx = fminf(fmaxf(fx, 0.f), (float)(w - 1));
    fy = fminf(fmaxf(fy, 0.f), (float)(h - 1));
    float x0f = floorf(fx), y0f = floorf(fy);
    BilinearTap t;
    t.x0 = (int)x0f; t.y0 = (int)y0f;
    t.x1 = t.x0 + 1 < w ? t.x0 + 1 : w - 1;
    t.y1 = t.y0 + 1 < h ? t.y0 + 1 : h - 1;
    t.wx = fx - x0f; t.wy = fy - y0f;
    return t;
}

// ---------------------------------------------------------------------------------------------------
// SE(3) exponential in double for pose <- exp(xi) * pose (PointRenderer.cu:1646-1657). Tangent order:
// translation part first, rotation part second. Host-and-device; libm sin/cos in double agree to the
// last bits that matter for a pose update (this one is compared with a tolerance, not bit-exactly).
// ---------------------------------------------------------------------------------------------------
ADOP_HD void se3_exp_left_multiply(const double* xi, double* pose8)
{
    double ux = xi[0], uy = xi[1], uz = xi[2];
    double wx = xi[3], wy = xi[4], wz = xi[5];
    double th2 = wx * wx + wy * wy + wz * wz;
    double th = sqrt(th2);
    // rotation quaternion of exp(w)
    double a, b;  // a = sin(th/2)/th , b = cos(th/2)
    double A, B;  // V = I + A W + B W^2 ; A = (1-cos)/th^2 , B = (th - sin)/th^3
    if (th < 1e-8)
    {
        a = 0.5 - th2 / 48.0; b = 1.0 - th2 / 8.0;
        A = 0.5 - th2 / 24.0; B = 1.0 / 6.0 - th2 / 120.0;
    }
    else
    {
        a = sin(0.5 * th) / th; b = cos(0.5 * th);
        A = (1.0 - cos(th)) / th2; B = (th - sin(th)) / (th2 * th);
    }
    double ex = a * wx, ey = a * wy, ez = a * wz, ew = b;
    // t_exp = V u = u + A (w x u) + B (w x (w x u))
    double c1x = wy * uz - wz * uy, c1y = wz * ux - wx * uz, c1z = wx * uy - wy * ux;
    double c2x = wy * c1z - wz * c1y, c2y = wz * c1x - wx * c1z, c2z = wx * c1y - wy * c1x;
    double tex = ux + A * c1x + B * c2x, tey = uy + A * c1y + B * c2y, tez = uz + A * c1z + B * c2z;
    // compose: q' = e * q ; t' = R(e) t + t_exp
    double qx = pose8[0], qy = pose8[1], qz = pose8[2], qw = pose8[3];
    double tx = pose8[4], ty = pose8[5], tz = pose8[6];
    double nx = ew * qx + ex * qw + ey * qz - ez * qy;
    double ny = ew * qy - ex * qz + ey * qw + ez * qx;
    double nz = ew * qz + ex * qy - ey * qx + ez * qw;
    double nw = ew * qw - ex * qx - ey * qy - ez * qz;
    double inorm = 1.0 / sqrt(nx * nx + ny * ny + nz * nz + nw * nw);
    // rotate t by e
    double uxx = 2.0 * (ey * tz - ez * ty), uyy = 2.0 * (ez * tx - ex * tz), uzz = 2.0 * (ex * ty - ey * tx);
    double rx = tx + ew * uxx + (ey * uzz - ez * uyy);
    double ry = ty + ew * uyy + (ez * uxx - ex * uzz);
    double rz = tz + ew * uzz + (ex * uyy - ey * uxx);
    pose8[0] = nx * inorm; pose8[1] = ny * inorm; pose8[2] = nz * inorm; pose8[3] = nw * inorm;
    pose8[4] = rx + tex; pose8[5] = ry + tey; pose8[6] = rz + tez;
}

}  // namespace adop
