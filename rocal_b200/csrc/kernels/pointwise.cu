// Pointwise family: window (crop) + flips + colour arithmetic + per-channel fma + layout/dtype
// conversion, one launch for the whole batch. grid = (tiles of the output extent, samples).
//
// Vector kernel (output width a multiple of 4, 16-byte aligned output): a thread owns 4 consecutive
// output pixels of one row. Their 12 source bytes are contiguous in the packed HWC source whatever
// the flips (a horizontal flip reverses the pixel order inside the block); they are fetched with
// four aligned 32-bit loads and three funnel shifts, so the arbitrary byte alignment of a 3-byte
// pixel row costs nothing, and leave as 16-byte (fp32), 8-byte (fp16) or 4-byte (uint8) stores.
// Work items (row, 4-pixel group) are flattened over the CTA so that widths that are not a multiple
// of the block size waste no lanes. The scalar kernel (one pixel per thread) covers other shapes.
//
// Colour arithmetic is float32 on the 0..255 scale with one rounding per operation:
//   brightness  y = alpha*x + beta
//   contrast    y = (x - center)*factor + center
//   twist       hexcone RGB->HSV with reciprocal multiplies (S = delta*(1/max),
//               H = 60*(num*(1/delta)) + offset; the reciprocals of the integer-valued delta and max
//               come from a 256-entry shared-memory table of IEEE 1/k), H += hue wrapped to [0,360),
//               S = clamp(S*sat,0,1), branch-free HSV->RGB  channel = V - V*S*clamp(min(k,4-k),0,1),
//               k = (n + H/60) mod 6, then alpha*x + beta
// The colour result is rounded to nearest even and saturated to uint8 before the optional
// normalisation (the reference's colour nodes output uint8 tensors).
#include "common.cuh"

namespace rb200 {

struct PointwiseLaunch {
    void* out;
    int out_w, out_h;
    int ext_w, ext_h;
    int tiles_x;
    int th;
    int color_op, normalize, fill_padding, reverse_channels;
    float mul[3], add[3];
    uint32_t magic;      // 0x4B000000, read by PRMT from the constant bank
    int pitch;           // vector kernel: bytes per staged source row (multiple of 16)
    int* status;         // vector kernel: written with 1 when the bounded wait on the staged rows gives up
    long long wait_cycles;   // vector kernel: limit of that wait, SM clock cycles
    int skip_row;        // vector kernel, self-test: the copy of this tile row is never issued (-1: all are)
    int overlap;         // vector kernel: 1 = independent of the preceding kernel, wait for it only before exit
    ArenaBounds bounds;  // bounds-checking build: the addresses the launch may read
};

__device__ __forceinline__ uint32_t pw_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool pw_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool pw_mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit) {
    if (pw_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < (1 << 24); i++) {
        if (pw_mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) break;
    }
    return false;
}

__device__ __forceinline__ float hsv_channel(float v, float vs, float hp, float nshift) {
    float k = add_rn(nshift, hp);
    if (k >= 6.f) k = sub_rn(k, 6.f);
    float t = fminf(k, sub_rn(4.f, k));
    t = fminf(fmaxf(t, 0.f), 1.f);
    return sub_rn(v, mul_rn(vs, t));
}

// rcp: table of 1/k for k = 0..255 (entry 0 holds 0).
__device__ __forceinline__ void color_twist_px(float r, float g, float b, float hue, float sat, const float* rcp,
                                               float& o0, float& o1, float& o2) {
    const float cmax = fmaxf(r, fmaxf(g, b));
    const float cmin = fminf(r, fminf(g, b));
    const float delta = sub_rn(cmax, cmin);
    // delta and cmax are integers in [0,255]: their low mantissa byte after adding 2^23 is the index
    const float rd = rcp[__float_as_uint(__fadd_rn(delta, 8388608.0f)) & 0xFFu];
    const float rm = rcp[__float_as_uint(__fadd_rn(cmax, 8388608.0f)) & 0xFFu];
    float s = mul_rn(delta, rm);
    const bool is_r = cmax == r;
    const bool is_g = cmax == g;
    const float num = is_r ? sub_rn(g, b) : (is_g ? sub_rn(b, r) : sub_rn(r, g));
    const float offs = is_r ? 0.f : (is_g ? 120.f : 240.f);
    float h = add_rn(mul_rn(60.f, mul_rn(num, rd)), offs);
    if (h < 0.f) h = add_rn(h, 360.f);
    h = add_rn(h, hue);
    h = sub_rn(h, mul_rn(360.f, floorf(mul_rn(h, 1.0f / 360.f))));
    s = mul_rn(s, sat);
    s = fminf(fmaxf(s, 0.f), 1.f);
    const float hp = mul_rn(h, 1.0f / 60.f);
    const float vs = mul_rn(cmax, s);
    o0 = hsv_channel(cmax, vs, hp, 5.f);
    o1 = hsv_channel(cmax, vs, hp, 3.f);
    o2 = hsv_channel(cmax, vs, hp, 1.f);
}

// ColorTwist of two pixels at once: the same operation sequence as color_twist_px followed by alpha*x + beta,
// with adds / multiplies that both pixels share issued as one packed f32x2 instruction (each lane rounds on
// its own, so a lane equals the scalar sequence) and the conditional corrections written as selects.
//
// A packed multiply whose result feeds a packed add or subtract is NOT safe: ptxas was measured to merge
// mul.rn.f32x2 + add.rn.f32x2 into one fused multiply-add (one rounding instead of two, whatever --fmad says),
// which moves a result across a rounding boundary about once in 10^5 values. A scalar add.rn of a packed
// product's lanes is never merged, so every such sum goes through lanes_add / lanes_sub.
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return fma2(b, make_float2(-1.0f, -1.0f), a); }   // a - b, one rounding
__device__ __forceinline__ float2 lanes_add(float2 a, float2 b) { return make_float2(add_rn(a.x, b.x), add_rn(a.y, b.y)); }
__device__ __forceinline__ float2 lanes_sub(float2 a, float2 b) { return make_float2(sub_rn(a.x, b.x), sub_rn(a.y, b.y)); }
__device__ __forceinline__ void color_twist_px2(float2 r, float2 g, float2 b, float alpha, float beta, float hue, float sat,
                                                const float* rcp, float2& o0, float2& o1, float2& o2) {
    float2 cmax, cmin;
    cmax.x = fmaxf(r.x, fmaxf(g.x, b.x)); cmax.y = fmaxf(r.y, fmaxf(g.y, b.y));
    cmin.x = fminf(r.x, fminf(g.x, b.x)); cmin.y = fminf(r.y, fminf(g.y, b.y));
    const float2 delta = sub2(cmax, cmin);
    const float2 k23 = make_float2(8388608.0f, 8388608.0f);
    const float2 di = add2(delta, k23), mi = add2(cmax, k23);     // integers 0..255 in the low mantissa byte
    float2 rd, rm;
    rd.x = rcp[__float_as_uint(di.x) & 0xFFu]; rd.y = rcp[__float_as_uint(di.y) & 0xFFu];
    rm.x = rcp[__float_as_uint(mi.x) & 0xFFu]; rm.y = rcp[__float_as_uint(mi.y) & 0xFFu];
    float2 s = mul2(delta, rm);
    const float2 gb = sub2(g, b), br = sub2(b, r), rg = sub2(r, g);
    float2 num, offs;
    {
        const bool ir = cmax.x == r.x, ig = cmax.x == g.x;
        num.x = ir ? gb.x : (ig ? br.x : rg.x);
        offs.x = ir ? 0.f : (ig ? 120.f : 240.f);
    }
    {
        const bool ir = cmax.y == r.y, ig = cmax.y == g.y;
        num.y = ir ? gb.y : (ig ? br.y : rg.y);
        offs.y = ir ? 0.f : (ig ? 120.f : 240.f);
    }
    float2 h = lanes_add(mul2(make_float2(60.f, 60.f), mul2(num, rd)), offs);
    const float2 hw = add2(h, make_float2(360.f, 360.f));
    h.x = h.x < 0.f ? hw.x : h.x;
    h.y = h.y < 0.f ? hw.y : h.y;
    h = add2(h, make_float2(hue, hue));
    float2 fl = mul2(h, make_float2(1.0f / 360.f, 1.0f / 360.f));
    fl.x = floorf(fl.x);
    fl.y = floorf(fl.y);
    h = lanes_sub(h, mul2(make_float2(360.f, 360.f), fl));
    s = mul2(s, make_float2(sat, sat));
    s.x = fminf(fmaxf(s.x, 0.f), 1.f);
    s.y = fminf(fmaxf(s.y, 0.f), 1.f);
    const float2 hp = mul2(h, make_float2(1.0f / 60.f, 1.0f / 60.f));
    const float2 vs = mul2(cmax, s);
    const float2 a2 = make_float2(alpha, alpha), b2 = make_float2(beta, beta);
    float2 out[3];
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const float nshift = c == 0 ? 5.f : (c == 1 ? 3.f : 1.f);
        float2 k = lanes_add(make_float2(nshift, nshift), hp);
        const float2 kw = add2(k, make_float2(-6.f, -6.f));
        k.x = k.x >= 6.f ? kw.x : k.x;
        k.y = k.y >= 6.f ? kw.y : k.y;
        const float2 k4 = sub2(make_float2(4.f, 4.f), k);
        float2 t;
        t.x = fminf(fmaxf(fminf(k.x, k4.x), 0.f), 1.f);
        t.y = fminf(fmaxf(fminf(k.y, k4.y), 0.f), 1.f);
        const float2 ch = lanes_sub(cmax, mul2(vs, t));
        out[c] = lanes_add(mul2(a2, ch), b2);
    }
    o0 = out[0];
    o1 = out[1];
    o2 = out[2];
}


// ---- RB200_ARITH_FAST: ColorTwist with fused operations, within one uint8 level of the exact sequence ----
// Internal operator code of the fast instantiation (not part of the C ABI).
constexpr int kColorTwistFast = 100;

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Per-sample constants of the fast path.
struct TwistFast {
    float2 hue_turns;     // hue / 360
    float2 sat;
    float a255, b255;     // alpha / 255, beta / 255: the affine step lands on the 0..1 scale so that .sat clamps it
};
__device__ __forceinline__ TwistFast twist_fast_setup(float alpha, float beta, float hue, float sat) {
    TwistFast t;
    const float ht = hue * (1.0f / 360.0f);
    t.hue_turns = make_float2(ht, ht);
    t.sat = make_float2(sat, sat);
    t.a255 = alpha * (1.0f / 255.0f);
    t.b255 = beta * (1.0f / 255.0f);
    return t;
}

// Two pixels (lanes x, y). The function is that of color_twist_px followed by alpha*x + beta, rearranged:
//   hue in turns  u = ((g-b | b-r | r-g) / delta + (0 | 2 | 4)) / 6 + hue/360      (one hardware reciprocal)
//   V*S           vs = clamp(delta * sat, 0, max)      (equal to max * clamp(delta/max * sat, 0, 1))
//   channel c     max - vs + vs * clamp(2 - 6 * |(u + K_c) - rint(u + K_c)|, 0, 1),  K = 1, 2/3, 1/3
// the last line being the periodic form of V - V*S*clamp(min(k, 4-k), 0, 1): no wrap-around selects are needed
// because the distance to the nearest integer is taken instead of a value modulo 6. Returns the three channels of both
// pixels as integers in the low mantissa byte of 1.5 * 2^23 + value.
__device__ __forceinline__ void color_twist_fast_px2(float2 r, float2 g, float2 b, const TwistFast& P, float2 (&o)[3]) {
    float2 cmax, cmin;
    cmax.x = fmaxf(r.x, fmaxf(g.x, b.x)); cmax.y = fmaxf(r.y, fmaxf(g.y, b.y));
    cmin.x = fminf(r.x, fminf(g.x, b.x)); cmin.y = fminf(r.y, fminf(g.y, b.y));
    const float2 neg1 = make_float2(-1.0f, -1.0f);
    const float2 delta = fma2(cmin, neg1, cmax);
    float2 rd;
    rd.x = rcp_approx(fmaxf(delta.x, 1e-20f));
    rd.y = rcp_approx(fmaxf(delta.y, 1e-20f));
    const float2 gb = fma2(b, neg1, g), br = fma2(r, neg1, b), rg = fma2(g, neg1, r);
    float2 num, offs;
    {
        const bool ir = cmax.x == r.x, ig = cmax.x == g.x;
        num.x = ir ? gb.x : (ig ? br.x : rg.x);
        offs.x = ir ? 0.f : (ig ? (2.0f / 6.0f) : (4.0f / 6.0f));
    }
    {
        const bool ir = cmax.y == r.y, ig = cmax.y == g.y;
        num.y = ir ? gb.y : (ig ? br.y : rg.y);
        offs.y = ir ? 0.f : (ig ? (2.0f / 6.0f) : (4.0f / 6.0f));
    }
    const float2 sixth = make_float2(1.0f / 6.0f, 1.0f / 6.0f);
    const float2 u0 = fma2(mul2(num, rd), sixth, add2(offs, P.hue_turns));
    float2 vs = mul2(delta, P.sat);
    vs.x = fminf(fmaxf(vs.x, 0.f), cmax.x);
    vs.y = fminf(fmaxf(vs.y, 0.f), cmax.y);
    const float2 vms = fma2(vs, neg1, cmax);
    const float2 big = make_float2(12582912.0f, 12582912.0f), nbig = make_float2(-12582912.0f, -12582912.0f);
    const float2 k255 = make_float2(255.0f, 255.0f);
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const float kc = c == 0 ? 1.0f : (c == 1 ? (2.0f / 3.0f) : (1.0f / 3.0f));
        const float2 uc = add2(u0, make_float2(kc, kc));
        const float2 ri = add2(add2(uc, big), nbig);            // nearest integer (|uc| is far below 2^22)
        const float2 fr = fma2(ri, neg1, uc);                   // in [-0.5, 0.5]
        float2 cc;
        cc.x = __saturatef(fmaf(-6.0f, fabsf(fr.x), 2.0f));
        cc.y = __saturatef(fmaf(-6.0f, fabsf(fr.y), 2.0f));
        const float2 ch = fma2(vs, cc, vms);
        float2 q;
        q.x = __saturatef(fmaf(P.a255, ch.x, P.b255));
        q.y = __saturatef(fmaf(P.a255, ch.y, P.b255));
        o[c] = fma2(q, k255, big);                              // round to nearest even, value in the low byte
    }
}

// The colour result before rounding and saturation.
template <int COLOR_OP>
__device__ __forceinline__ void color_raw(float& v0, float& v1, float& v2, float alpha, float beta, float hue, float sat,
                                          const float* rcp) {
    if (COLOR_OP == RB200_COLOR_BRIGHTNESS) {
        v0 = add_rn(mul_rn(alpha, v0), add_rn(beta, hue));     // hue = 0 unless the offset is tilted (colour temperature)
        v1 = add_rn(mul_rn(alpha, v1), beta);
        v2 = add_rn(mul_rn(alpha, v2), sub_rn(beta, hue));
    } else if (COLOR_OP == RB200_COLOR_GAMMA) {
        v0 = mul_rn(255.0f, powf(mul_rn(v0, 1.0f / 255.0f), alpha));
        v1 = mul_rn(255.0f, powf(mul_rn(v1, 1.0f / 255.0f), alpha));
        v2 = mul_rn(255.0f, powf(mul_rn(v2, 1.0f / 255.0f), alpha));
    } else if (COLOR_OP == RB200_COLOR_CONTRAST) {
        v0 = add_rn(mul_rn(sub_rn(v0, beta), alpha), beta);
        v1 = add_rn(mul_rn(sub_rn(v1, beta), alpha), beta);
        v2 = add_rn(mul_rn(sub_rn(v2, beta), alpha), beta);
    } else if (COLOR_OP == RB200_COLOR_TWIST || COLOR_OP == kColorTwistFast) {
        float t0, t1, t2;
        color_twist_px(v0, v1, v2, hue, sat, rcp, t0, t1, t2);
        v0 = add_rn(mul_rn(alpha, t0), beta);
        v1 = add_rn(mul_rn(alpha, t1), beta);
        v2 = add_rn(mul_rn(alpha, t2), beta);
    }
}

template <int COLOR_OP>
__device__ __forceinline__ void color_px(float& v0, float& v1, float& v2, float alpha, float beta, float hue, float sat,
                                         const float* rcp) {
    if (COLOR_OP != RB200_COLOR_NONE) {
        color_raw<COLOR_OP>(v0, v1, v2, alpha, beta, hue, sat, rcp);
        v0 = sat_round_u8f(v0);
        v1 = sat_round_u8f(v1);
        v2 = sat_round_u8f(v2);
    }
}

// Round to nearest even and saturate to [0,255] in one conversion (NaN gives 0): the same result as
// sat_round_u8f, as an integer.
__device__ __forceinline__ uint32_t cvt_sat_u8(float v) {
    uint32_t r;
    asm("cvt.rni.u8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ uint32_t pack4_u8(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040u), __byte_perm(c, d, 0x0040u), 0x5410u);
}

template <typename OutT, int LAYOUT>
__device__ __forceinline__ void pw_store3(OutT* out, int out_w, int out_h, int n, int y, int x, float v0, float v1, float v2) {
    if (LAYOUT == RB200_NCHW) {
        size_t plane = (size_t)out_w * out_h;
        size_t base = ((size_t)n * 3) * plane + (size_t)y * out_w + x;
        out[base] = OutConv<OutT>::cvt(v0);
        out[base + plane] = OutConv<OutT>::cvt(v1);
        out[base + 2 * plane] = OutConv<OutT>::cvt(v2);
    } else {
        size_t base = (((size_t)n * out_h + y) * out_w + x) * 3;
        out[base] = OutConv<OutT>::cvt(v0);
        out[base + 1] = OutConv<OutT>::cvt(v1);
        out[base + 2] = OutConv<OutT>::cvt(v2);
    }
}

// Four consecutive elements of one type, stored as one vector.
template <typename OutT>
struct Store4;
template <>
struct Store4<float> {
    static __device__ __forceinline__ void st(float* p, float a, float b, float c, float d) {
        *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    }
};
template <>
struct Store4<__half> {
    static __device__ __forceinline__ void st(__half* p, float a, float b, float c, float d) {
        __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
        uint2 v;
        v.x = *reinterpret_cast<uint32_t*>(&lo);
        v.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = v;
    }
};
template <>
struct Store4<uint8_t> {
    // Inputs are integer valued in [0,255]: adding 2^23 leaves the value in the low mantissa byte.
    static __device__ __forceinline__ void st(uint8_t* p, float a, float b, float c, float d) {
        uint32_t ab = __byte_perm(__float_as_uint(__fadd_rn(a, 8388608.0f)), __float_as_uint(__fadd_rn(b, 8388608.0f)), 0x0040u);
        uint32_t cd = __byte_perm(__float_as_uint(__fadd_rn(c, 8388608.0f)), __float_as_uint(__fadd_rn(d, 8388608.0f)), 0x0040u);
        *reinterpret_cast<uint32_t*>(p) = __byte_perm(ab, cd, 0x5410u);
    }
};

// Byte-only path of crop / flip for uint8 output: the 12 source bytes d[0..2] of a 4-pixel block are
// permuted into the three output words without ever becoming floats.
template <int LAYOUT>
__device__ __forceinline__ void permute_store_u8(uint8_t* po, size_t plane, const uint32_t (&d)[3], bool flip) {
    if (LAYOUT == RB200_NHWC) {
        uint32_t o0 = d[0], o1 = d[1], o2 = d[2];
        if (flip) {   // pixel order reversed, channel order kept
            o0 = __byte_perm(d[1], d[2], 0x2765u);
            o1 = __byte_perm(__byte_perm(d[1], d[2], 0x0043u), d[0], 0x3710u);
            o2 = __byte_perm(d[0], d[1], 0x2105u);
        }
        reinterpret_cast<uint32_t*>(po)[0] = o0;
        reinterpret_cast<uint32_t*>(po)[1] = o1;
        reinterpret_cast<uint32_t*>(po)[2] = o2;
    } else {
        // channel c of pixels 0..3 = block bytes c, 3+c, 6+c, 9+c
        uint32_t r = __byte_perm(__byte_perm(d[0], d[1], 0x0630u), d[2], 0x5210u);
        uint32_t g = __byte_perm(__byte_perm(d[0], d[1], 0x0741u), d[2], 0x6210u);
        uint32_t b = __byte_perm(__byte_perm(d[0], d[1], 0x0052u), d[2], 0x7410u);
        // b: bytes 2, 5, 8, 11 = d[0].2, d[1].1, d[2].0, d[2].3
        if (flip) {
            r = __byte_perm(r, 0u, 0x0123u);
            g = __byte_perm(g, 0u, 0x0123u);
            b = __byte_perm(b, 0u, 0x0123u);
        }
        *reinterpret_cast<uint32_t*>(po) = r;
        *reinterpret_cast<uint32_t*>(po + plane) = g;
        *reinterpret_cast<uint32_t*>(po + 2 * plane) = b;
    }
}

// uint8 in, uint8 out colour operators on one 4-pixel block: d[] are the 12 source bytes, e[] the 12 result
// bytes in the same (block) order. COLOR_NONE copies.
template <int COLOR_OP>
__device__ __forceinline__ void color_block_u8(const uint32_t (&d)[3], uint32_t (&e)[3], uint32_t magic, float alpha, float beta,
                                               float hue, float sat, const float* rcp) {
    if (COLOR_OP == RB200_COLOR_NONE) {
        e[0] = d[0]; e[1] = d[1]; e[2] = d[2];
    } else if (COLOR_OP == kColorTwistFast) {
        const TwistFast P = twist_fast_setup(alpha, beta, hue, sat);
        const float2 nk23 = make_float2(-8388608.0f, -8388608.0f);
        uint32_t q[12];
#pragma unroll
        for (int k = 0; k < 4; k += 2) {
            float2 c3[3];
#pragma unroll
            for (int c = 0; c < 3; c++) {
                const int ba = 3 * k + c, bb = 3 * (k + 1) + c;
                c3[c].x = __uint_as_float(__byte_perm(d[ba >> 2], magic, 0x7650u + (ba & 3)));
                c3[c].y = __uint_as_float(__byte_perm(d[bb >> 2], magic, 0x7650u + (bb & 3)));
                c3[c] = add2(c3[c], nk23);
            }
            float2 o[3];
            color_twist_fast_px2(c3[0], c3[1], c3[2], P, o);
#pragma unroll
            for (int c = 0; c < 3; c++) {
                q[3 * k + c] = __float_as_uint(o[c].x);
                q[3 * k + 3 + c] = __float_as_uint(o[c].y);
            }
        }
#pragma unroll
        for (int wd = 0; wd < 3; wd++)
            e[wd] = __byte_perm(__byte_perm(q[4 * wd], q[4 * wd + 1], 0x0040u), __byte_perm(q[4 * wd + 2], q[4 * wd + 3], 0x0040u), 0x5410u);
    } else if (COLOR_OP == RB200_COLOR_TWIST) {
        uint32_t q[12];
        const float2 nk23 = make_float2(-8388608.0f, -8388608.0f);
#pragma unroll
        for (int k = 0; k < 4; k += 2) {       // pixels k and k+1 of the block in the two lanes
            float2 c3[3];
#pragma unroll
            for (int c = 0; c < 3; c++) {
                const int ba = 3 * k + c, bb = 3 * (k + 1) + c;
                c3[c].x = __uint_as_float(__byte_perm(d[ba >> 2], magic, 0x7650u + (ba & 3)));
                c3[c].y = __uint_as_float(__byte_perm(d[bb >> 2], magic, 0x7650u + (bb & 3)));
                c3[c] = add2(c3[c], nk23);
            }
            float2 o0, o1, o2;
            color_twist_px2(c3[0], c3[1], c3[2], alpha, beta, hue, sat, rcp, o0, o1, o2);
            q[3 * k + 0] = cvt_sat_u8(o0.x); q[3 * k + 1] = cvt_sat_u8(o1.x); q[3 * k + 2] = cvt_sat_u8(o2.x);
            q[3 * k + 3] = cvt_sat_u8(o0.y); q[3 * k + 4] = cvt_sat_u8(o1.y); q[3 * k + 5] = cvt_sat_u8(o2.y);
        }
#pragma unroll
        for (int wd = 0; wd < 3; wd++) e[wd] = pack4_u8(q[4 * wd], q[4 * wd + 1], q[4 * wd + 2], q[4 * wd + 3]);
    } else {
        // brightness / contrast: two bytes per packed f32x2 instruction
        const float2 nk23 = make_float2(-8388608.0f, -8388608.0f);
        const float2 a2 = make_float2(alpha, alpha), b2 = make_float2(beta, beta);
        const float2 nb2 = make_float2(-beta, -beta);
        // brightness: the offset of channel c (byte index mod 3) is beta + hue, beta, beta - hue
        const float bc[3] = {add_rn(beta, hue), beta, sub_rn(beta, hue)};
#pragma unroll
        for (int wd = 0; wd < 3; wd++) {
            uint32_t q[4];
#pragma unroll
            for (int hb = 0; hb < 4; hb += 2) {
                float2 x;
                x.x = __uint_as_float(__byte_perm(d[wd], magic, 0x7650u + hb));
                x.y = __uint_as_float(__byte_perm(d[wd], magic, 0x7651u + hb));
                x = add2(x, nk23);
                if (COLOR_OP == RB200_COLOR_BRIGHTNESS)
                    x = lanes_add(mul2(a2, x), make_float2(bc[(4 * wd + hb) % 3], bc[(4 * wd + hb + 1) % 3]));
                else
                    x = lanes_add(mul2(add2(x, nb2), a2), b2);
                q[hb] = cvt_sat_u8(x.x);
                q[hb + 1] = cvt_sat_u8(x.y);
            }
            e[wd] = pack4_u8(q[0], q[1], q[2], q[3]);
        }
    }
}

template <typename OutT, int LAYOUT, int COLOR_OP>
// Every instantiation is bound by latency (a CTA waits once for its staged rows) as much as by issue, so the minimum
// number of resident CTAs per SM is asked for explicitly. ColorTwist: six (40 registers) measured 37 / 27 us per
// 256-image launch (exact / fast arithmetic) against 51 / 33 us at the register count the compiler picks on its own
// (122 / 70: two or three CTAs per SM). The others: seven (32 registers, a few dozen bytes of spills in some) measured
// 15.5 us (brightness) and 15.4 us (flip) against 21.9 / 19.1 us at the compiler's 48-50 registers.
__global__ void __launch_bounds__(256, (COLOR_OP == kColorTwistFast || COLOR_OP == RB200_COLOR_TWIST) ? 6 : 7) pointwise_vec_kernel(const uint8_t* __restrict__ arena,
                                                            const rb200_pointwise_sample* __restrict__ samples,
                                                            const PointwiseLaunch L) {
    // Layout: mbarrier (16 bytes) | rcp[256] | staged source rows (th x pitch)
    extern __shared__ __align__(16) uint8_t pw_smem[];
    __shared__ int stage_flag;
    pdl_launch_dependents();
    float* rcp = reinterpret_cast<float*>(pw_smem + 16);
    // the reciprocal table depends on nothing in memory: it is built while the preceding kernel drains
    if (COLOR_OP == RB200_COLOR_TWIST || COLOR_OP == kColorTwistFast)
        for (int k = threadIdx.x; k < 256; k += blockDim.x) rcp[k] = k ? div_rn(1.0f, (float)k) : 0.f;
    if (!L.overlap) pdl_wait();
    uint8_t* stage = pw_smem + 16 + 1024;
    const uint32_t bar = pw_smem_u32(pw_smem);
    const int n = blockIdx.y;
    const int tile_y0 = blockIdx.x * L.th;
    const rb200_pointwise_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);
    const int w = min(s.roi_w, L.out_w);
    const int h = min(s.roi_h, L.out_h);
    // bounds-checking build: a sample whose window leaves the arena is reported and none of it is read
    const bool src_ok = rect_in_bounds(L.bounds, img, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status);
    const int rows = src_ok ? min(L.th, h - tile_y0) : 0;
    const size_t plane = (size_t)L.out_w * L.out_h;
    // first source column of every row of the window (a horizontal flip shows the last w columns)
    const int x_src0 = s.flip_h ? (s.roi_x + s.roi_w - w) : s.roi_x;
    bool staged_ok = true;

    if (rows > 0 && w > 0) {
        // Stage the tile's source rows: lane r of warp 0 issues one bulk copy per row r, r+32, ...
        if (threadIdx.x == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(min(rows, 32)) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();
        if (threadIdx.x < 32 && (int)threadIdx.x < rows) {
            uint32_t total = 0;
            for (int r = threadIdx.x; r < rows; r += 32) {
                const int y = tile_y0 + r;
                const int sy = s.roi_y + (s.flip_v ? (s.roi_h - 1 - y) : y);
                const uint8_t* g = img + (size_t)sy * s.src_stride + (size_t)x_src0 * 3;
                const uint32_t m = (uint32_t)((uintptr_t)g & 15);
                total += ((m + (uint32_t)w * 3 + 15) >> 4) << 4;
            }
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
            for (int r = threadIdx.x; r < rows; r += 32) {
                const int y = tile_y0 + r;
                const int sy = s.roi_y + (s.flip_v ? (s.roi_h - 1 - y) : y);
                const uint8_t* g = img + (size_t)sy * s.src_stride + (size_t)x_src0 * 3;
                const uint32_t m = (uint32_t)((uintptr_t)g & 15);
                const uint32_t bytes = ((m + (uint32_t)w * 3 + 15) >> 4) << 4;
                if (r == L.skip_row) continue;     // self-test: this row's bytes stay expected and never arrive
                if (!span_in_bounds(L.bounds, g - m, bytes, L.status)) continue;   // (bounds-checking build)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(pw_smem_u32(stage + (size_t)r * L.pitch)), "l"(g - m), "r"(bytes), "r"(bar) : "memory");
            }
        }
        // Warp 0 waits for the copies (bounded); the other warps sleep at the barrier instead of polling.
        if (threadIdx.x < 32) {
            const bool ok = pw_mbar_wait_bounded(bar, 0, L.wait_cycles);
            if (threadIdx.x == 0) {
                stage_flag = ok ? 1 : 0;
                if (!ok) {
                    raise_status(L.status);
                    pw_mbar_wait_bounded(bar, 0, L.wait_cycles);   // second bounded chance for copies still in flight
                }
            }
        }
        __syncthreads();
        staged_ok = stage_flag != 0;
    }

    if (rows > 0 && w > 0 && staged_ok) {
        const bool bytes_only = COLOR_OP == RB200_COLOR_NONE && sizeof(OutT) == 1 && !L.normalize && !L.reverse_channels;
        // uint8 NHWC output without normalisation: the first w16 columns of every row go through 16-pixel units
        // (48 source bytes -> 48 output bytes per thread and step), which spreads the index arithmetic of an
        // item over four 4-pixel blocks and lets the result leave as three 16-byte stores; the item loop below
        // takes the remaining columns (and everything for the other output types).
        const bool unit_path = sizeof(OutT) == 1 && LAYOUT == RB200_NHWC && !L.normalize && !L.reverse_channels &&
                               COLOR_OP != RB200_COLOR_GAMMA;
        const int w16 = unit_path ? (w & ~15) : 0;
        const int gpr = (w - w16 + 3) >> 2;           // 4-pixel groups per row in the item loop
        const int items = rows * gpr;
        // item / gpr by multiply-high: exact while item * gpr < 2^32
        const uint32_t gpr_magic = gpr > 0 ? (uint32_t)((0x100000000ull + (uint32_t)gpr - 1) / (uint32_t)gpr) : 0u;
        // Per-thread constants of the index arithmetic: source row of tile row r is sy0 + sy_step * r; a
        // staged row starts at the source row's address rounded down to 16 bytes, so the block of group
        // column x sits at (row address mod 16) + 3 * (x, or w - x - npx under a horizontal flip).
        const int sy0 = s.roi_y + (s.flip_v ? (s.roi_h - 1 - tile_y0) : tile_y0);
        const int sy_step = s.flip_v ? -1 : 1;
        const uint32_t base_mod = (uint32_t)((uintptr_t)(img + (size_t)x_src0 * 3) & 15);
        const uint32_t stride_mod = s.src_stride & 15;
        // element (tile row 0, column 0) of the output; an item adds a 32-bit offset
        OutT* const out_tile = out + (LAYOUT == RB200_NCHW ? ((size_t)n * 3) * plane + (size_t)tile_y0 * L.out_w
                                                             : ((size_t)n * L.out_h + tile_y0) * L.out_w * 3);
        if (w16 > 0) {
            const int upr = w16 >> 4;
            const int units = rows * upr;
            const uint32_t upr_div = (uint32_t)(upr > 0 ? upr : 1);     // upr >= 1 here; spelled out for instantiations where w16 folds to 0
            const uint32_t upr_magic = (uint32_t)((0x100000000ull + upr_div - 1) / upr_div);
            uint8_t* const out_bytes = reinterpret_cast<uint8_t*>(out_tile);
            const bool st16 = ((reinterpret_cast<uintptr_t>(out_bytes) | (uintptr_t)(L.out_w * 3)) & 15u) == 0;
            for (int unit = threadIdx.x; unit < units; unit += blockDim.x) {
                const int row = upr == 1 ? unit : (int)__umulhi((uint32_t)unit, upr_magic);
                const int x = (unit - row * upr) << 4;
                const int sy = sy0 + sy_step * row;
                const uint32_t m = (base_mod + (uint32_t)sy * stride_mod) & 15u;
                const uint32_t boff = (uint32_t)row * L.pitch + m + (uint32_t)(s.flip_h ? (w - x - 16) : x) * 3u;
                const uint32_t* wp = reinterpret_cast<const uint32_t*>(stage + (boff & ~3u));
                uint32_t wv[13];
#pragma unroll
                for (int i = 0; i < 13; i++) wv[i] = wp[i];
                const uint32_t sh = boff << 3;          // the funnel shift reads the low five bits
                uint32_t ee[12];
#pragma unroll
                for (int b = 0; b < 4; b++) {           // source block b = source pixels 4b .. 4b+3 of the unit
                    uint32_t d[3], e[3];
                    d[0] = __funnelshift_r(wv[3 * b], wv[3 * b + 1], sh);
                    d[1] = __funnelshift_r(wv[3 * b + 1], wv[3 * b + 2], sh);
                    d[2] = __funnelshift_r(wv[3 * b + 2], wv[3 * b + 3], sh);
                    color_block_u8<COLOR_OP>(d, e, L.magic, s.alpha, s.beta, s.hue, s.sat, rcp);
                    if (s.flip_h) {                     // blocks and the pixels inside a block change places
                        ee[3 * (3 - b) + 0] = __byte_perm(e[1], e[2], 0x2765u);
                        ee[3 * (3 - b) + 1] = __byte_perm(__byte_perm(e[1], e[2], 0x0043u), e[0], 0x3710u);
                        ee[3 * (3 - b) + 2] = __byte_perm(e[0], e[1], 0x2105u);
                    } else {
                        ee[3 * b + 0] = e[0]; ee[3 * b + 1] = e[1]; ee[3 * b + 2] = e[2];
                    }
                }
                uint8_t* po = out_bytes + (uint32_t)(row * L.out_w + x) * 3u;
                if (st16) {
#pragma unroll
                    for (int q = 0; q < 3; q++)
                        reinterpret_cast<uint4*>(po)[q] = make_uint4(ee[4 * q], ee[4 * q + 1], ee[4 * q + 2], ee[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 12; q++) reinterpret_cast<uint32_t*>(po)[q] = ee[q];
                }
            }
        }
        // Two work items per iteration: all eight loads are issued before the first use.
        for (int item0 = threadIdx.x; item0 < items; item0 += 2 * blockDim.x) {
            uint32_t wv[2][4];
            uint32_t shv[2];
            int xv[2], yv[2], npxv[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int item = item0 + u * blockDim.x;
                npxv[u] = 0;
                if (item < items) {
                    const int row = gpr == 1 ? item : (int)__umulhi((uint32_t)item, gpr_magic);
                    const int x = w16 + ((item - row * gpr) << 2);
                    const int npx = min(4, w - x);
                    const int sy = sy0 + sy_step * row;
                    const uint32_t m = (base_mod + (uint32_t)sy * stride_mod) & 15u;
                    const uint32_t boff = (uint32_t)row * L.pitch + m + (uint32_t)(s.flip_h ? (w - x - npx) : x) * 3u;
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(stage + (boff & ~3u));
                    wv[u][0] = wp[0];
                    wv[u][1] = wp[1];
                    wv[u][2] = wp[2];
                    wv[u][3] = wp[3];
                    shv[u] = boff << 3;      // the funnel shift reads the low five bits
                    xv[u] = x; yv[u] = tile_y0 + row; npxv[u] = npx;
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int npx = npxv[u];
                if (npx == 0) continue;
                const int x = xv[u], y = yv[u];
                // element offset of the block's first output pixel inside the tile
                const uint32_t eoff = (uint32_t)((y - tile_y0) * L.out_w + x) * (LAYOUT == RB200_NCHW ? 1u : 3u);
                uint32_t d[3];
                d[0] = __funnelshift_r(wv[u][0], wv[u][1], shv[u]);
                d[1] = __funnelshift_r(wv[u][1], wv[u][2], shv[u]);
                d[2] = __funnelshift_r(wv[u][2], wv[u][3], shv[u]);
                if (bytes_only && npx == 4) {
                    uint8_t* pb = reinterpret_cast<uint8_t*>(out_tile) + eoff;
                    permute_store_u8<LAYOUT>(pb, plane, d, s.flip_h != 0);
                    continue;
                }
                if (COLOR_OP != RB200_COLOR_NONE && COLOR_OP != RB200_COLOR_GAMMA && sizeof(OutT) == 1 && !L.normalize &&
                    !L.reverse_channels && npx == 4) {
                    // uint8 in, uint8 out: the 12 result bytes are rebuilt in block order and leave through the
                    // same byte permutation as a plain crop / flip.
                    uint32_t e[3];
                    color_block_u8<COLOR_OP>(d, e, L.magic, s.alpha, s.beta, s.hue, s.sat, rcp);
                    uint8_t* pb = reinterpret_cast<uint8_t*>(out_tile) + eoff;
                    permute_store_u8<LAYOUT>(pb, plane, e, s.flip_h != 0);
                    continue;
                }
                // block pixel k, channel c = byte 3k+c of d[]
                float v[4][3];
#pragma unroll
                for (int k = 0; k < 4; k++) {
#pragma unroll
                    for (int c = 0; c < 3; c++) {
                        const int bidx = 3 * k + c;
                        v[k][c] = sub_rn(__uint_as_float(__byte_perm(d[bidx >> 2], L.magic, 0x7650u + (bidx & 3))), 8388608.0f);
                    }
                    color_px<COLOR_OP>(v[k][0], v[k][1], v[k][2], s.alpha, s.beta, s.hue, s.sat, rcp);
                    if (L.reverse_channels) { float t = v[k][0]; v[k][0] = v[k][2]; v[k][2] = t; }
                    if (L.normalize) {
                        v[k][0] = fmaf(v[k][0], L.mul[0], L.add[0]);
                        v[k][1] = fmaf(v[k][1], L.mul[1], L.add[1]);
                        v[k][2] = fmaf(v[k][2], L.mul[2], L.add[2]);
                    }
                }
                if (npx == 4) {
                    // output pixel j shows block pixel (flip_h ? 3-j : j)
                    float o[4][3];
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int c = 0; c < 3; c++) {
                            o[j][c] = s.flip_h ? v[3 - j][c] : v[j][c];
                            if (sizeof(OutT) == 1 && L.normalize) o[j][c] = sat_round_u8f(o[j][c]);
                        }
                    if (LAYOUT == RB200_NCHW) {
                        OutT* po = out_tile + eoff;
                        Store4<OutT>::st(po, o[0][0], o[1][0], o[2][0], o[3][0]);
                        Store4<OutT>::st(po + plane, o[0][1], o[1][1], o[2][1], o[3][1]);
                        Store4<OutT>::st(po + 2 * plane, o[0][2], o[1][2], o[2][2], o[3][2]);
                    } else {
                        OutT* po = out_tile + eoff;
                        Store4<OutT>::st(po, o[0][0], o[0][1], o[0][2], o[1][0]);
                        Store4<OutT>::st(po + 4, o[1][1], o[1][2], o[2][0], o[2][1]);
                        Store4<OutT>::st(po + 8, o[2][2], o[3][0], o[3][1], o[3][2]);
                    }
                } else {
                    for (int j = 0; j < npx; j++) {
                        const int k = s.flip_h ? (npx - 1 - j) : j;
                        float a = k == 0 ? v[0][0] : (k == 1 ? v[1][0] : v[2][0]);
                        float b = k == 0 ? v[0][1] : (k == 1 ? v[1][1] : v[2][1]);
                        float c = k == 0 ? v[0][2] : (k == 1 ? v[1][2] : v[2][2]);
                        pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, x + j, a, b, c);
                    }
                }
            }
        }
    }
    if (L.fill_padding && (w < L.out_w || h < L.out_h)) {
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int item = threadIdx.x; item < rows_in_tile * L.out_w; item += blockDim.x) {
            const int row = item / L.out_w;
            const int x = item - row * L.out_w;
            const int y = tile_y0 + row;
            if (y >= h || x >= w) pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, x, 0.f, 0.f, 0.f);
        }
    }
    if (L.overlap) pdl_wait();      // completion of this launch implies completion of the kernel before it
}

// Scalar kernel: one thread per output column, any width and alignment.
template <typename OutT, int LAYOUT, int COLOR_OP>
__global__ void __launch_bounds__(256) pointwise_kernel(const uint8_t* __restrict__ arena,
                                                        const rb200_pointwise_sample* __restrict__ samples,
                                                        const PointwiseLaunch L) {
    __shared__ float rcp[256];
    if (COLOR_OP == RB200_COLOR_TWIST) {
        for (int k = threadIdx.x; k < 256; k += blockDim.x) rcp[k] = k ? div_rn(1.0f, (float)k) : 0.f;
        __syncthreads();
    }
    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int xi = tx * blockDim.x + threadIdx.x;
    const int tile_y0 = ty * L.th;

    const rb200_pointwise_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);
    const int w = min(s.roi_w, L.out_w);
    const int h = min(s.roi_h, L.out_h);
    // (bounds-checking build; the second image of a blend may live in another allocation and is not checked)
    const bool src_ok = rect_in_bounds(L.bounds, img, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status);

    if (xi < w && src_ok) {
        const int sx = s.roi_x + (s.flip_h ? (s.roi_w - 1 - xi) : xi);
        const int rows = min(L.th, h - tile_y0);
        for (int j = 0; j < rows; j++) {
            const int y = tile_y0 + j;
            const int sy = s.roi_y + (s.flip_v ? (s.roi_h - 1 - y) : y);
            const uint8_t* px = img + (size_t)sy * s.src_stride + (size_t)sx * 3;
            float v0 = (float)__ldg(px), v1 = (float)__ldg(px + 1), v2 = (float)__ldg(px + 2);
            if (COLOR_OP == RB200_COLOR_BLEND) {
                // the same pixel of the second source: alpha*x + (1 - alpha)*x2, rounded and saturated
                const uint8_t* img2 = arena + (((uint64_t)s.src2_offset_hi << 32) | s.src2_offset_lo);
                const uint8_t* p2 = img2 + (size_t)sy * s.src2_stride + (size_t)sx * 3;
                const float w2 = sub_rn(1.0f, s.alpha);
                v0 = sat_round_u8f(add_rn(mul_rn(s.alpha, v0), mul_rn(w2, (float)__ldg(p2))));
                v1 = sat_round_u8f(add_rn(mul_rn(s.alpha, v1), mul_rn(w2, (float)__ldg(p2 + 1))));
                v2 = sat_round_u8f(add_rn(mul_rn(s.alpha, v2), mul_rn(w2, (float)__ldg(p2 + 2))));
            } else {
                color_px<COLOR_OP>(v0, v1, v2, s.alpha, s.beta, s.hue, s.sat, rcp);
            }
            if (L.reverse_channels) { float t = v0; v0 = v2; v2 = t; }
            if (L.normalize) {
                v0 = fmaf(v0, L.mul[0], L.add[0]);
                v1 = fmaf(v1, L.mul[1], L.add[1]);
                v2 = fmaf(v2, L.mul[2], L.add[2]);
            }
            pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, v0, v1, v2);
        }
    }
    if (L.fill_padding && xi < L.out_w) {
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int j = 0; j < rows_in_tile; j++) {
            int y = tile_y0 + j;
            if (y >= h || xi >= w) pw_store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
        }
    }
}

template <typename OutT, int LAYOUT, int COLOR_OP>
static void launch_one(bool vec, dim3 grid, int threads, size_t smem, cudaStream_t stream, const uint8_t* arena,
                       const rb200_pointwise_sample* samples, const PointwiseLaunch& L) {
    if (vec) {
        auto k = pointwise_vec_kernel<OutT, LAYOUT, COLOR_OP>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_overlapped(k, grid, dim3((unsigned)threads), smem, stream, arena, samples, L);
    } else
        pointwise_kernel<OutT, LAYOUT, COLOR_OP><<<grid, threads, 0, stream>>>(arena, samples, L);
}

template <typename OutT, int LAYOUT>
static int launch_color(int color_op, bool vec, dim3 grid, int threads, size_t smem, cudaStream_t stream, const uint8_t* arena,
                        const rb200_pointwise_sample* samples, const PointwiseLaunch& L) {
    switch (color_op) {
        case RB200_COLOR_NONE: launch_one<OutT, LAYOUT, RB200_COLOR_NONE>(vec, grid, threads, smem, stream, arena, samples, L); break;
        case RB200_COLOR_BRIGHTNESS: launch_one<OutT, LAYOUT, RB200_COLOR_BRIGHTNESS>(vec, grid, threads, smem, stream, arena, samples, L); break;
        case RB200_COLOR_CONTRAST: launch_one<OutT, LAYOUT, RB200_COLOR_CONTRAST>(vec, grid, threads, smem, stream, arena, samples, L); break;
        case RB200_COLOR_TWIST: launch_one<OutT, LAYOUT, RB200_COLOR_TWIST>(vec, grid, threads, smem, stream, arena, samples, L); break;
        case kColorTwistFast:
            // only the uint8 vector kernel has a fast block; every other shape was routed to the exact operator
            launch_one<OutT, LAYOUT, sizeof(OutT) == 1 ? kColorTwistFast : RB200_COLOR_TWIST>(true, grid, threads, smem, stream, arena, samples, L);
            break;
        case RB200_COLOR_GAMMA: launch_one<OutT, LAYOUT, RB200_COLOR_GAMMA>(vec, grid, threads, smem, stream, arena, samples, L); break;
        case RB200_COLOR_BLEND:   // two sources: the scalar kernel only
            pointwise_kernel<OutT, LAYOUT, RB200_COLOR_BLEND><<<grid, threads, 0, stream>>>(arena, samples, L);
            break;
        default: set_error("rb200k_pointwise: bad color_op %d", color_op); return RB200_E_INVALID;
    }
    RB200_CHECK_LAUNCH("pointwise_kernel");
    return RB200_OK;
}

}  // namespace rb200

using namespace rb200;

static int pointwise_launch(const uint8_t* arena, const rb200_pointwise_sample* samples,
                            const rb200_pointwise_sample* h_samples, int n, const rb200_pointwise_params* p,
                            void* stream_v, unsigned long long wait_cycles, int skip_row) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_pointwise: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_pointwise: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (p->out_dtype < 0 || p->out_dtype > 2 || (p->out_layout != RB200_NCHW && p->out_layout != RB200_NHWC)) {
        set_error("rb200k_pointwise: bad out_dtype %d / out_layout %d", p->out_dtype, p->out_layout);
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;
    PointwiseLaunch L;
    L.out = p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.color_op = p->color_op;
    L.normalize = p->normalize;
    L.fill_padding = p->fill_padding;
    L.reverse_channels = p->reverse_channels;
    L.magic = 0x4B000000u;
    for (int c = 0; c < 3; c++) { L.mul[c] = p->mul[c]; L.add[c] = p->add[c]; }
    if (p->arith != RB200_ARITH_EXACT && p->arith != RB200_ARITH_FAST) {
        set_error("rb200k_pointwise: bad arith %d", p->arith);
        return RB200_E_INVALID;
    }
    L.status = p->status ? p->status : default_status_word();
    if (!L.status) {
        set_error("rb200k_pointwise: the device's status word cannot be addressed");
        return RB200_E_CUDA;
    }
    L.wait_cycles = (long long)(wait_cycles ? wait_cycles : kDefaultWaitCycles);
    L.skip_row = skip_row;
    L.overlap = p->overlap ? 1 : 0;
    L.bounds = arena_bounds(arena, p->arena_bytes);
    if (p->out_bytes && (uint64_t)n * p->out_w * p->out_h * 3 * out_elem_size(p->out_dtype) > p->out_bytes) {
        set_error("rb200k_pointwise: %d samples of %d x %d x 3 elements do not fit the %llu-byte output", n, p->out_w, p->out_h,
                  (unsigned long long)p->out_bytes);
        return RB200_E_INVALID;
    }
    int ext_w = p->out_w, ext_h = p->out_h;
    if (h_samples && !p->fill_padding) {
        ext_w = 1; ext_h = 1;
        for (int i = 0; i < n; i++) {
            int w = h_samples[i].roi_w < p->out_w ? h_samples[i].roi_w : p->out_w;
            int h = h_samples[i].roi_h < p->out_h ? h_samples[i].roi_h : p->out_h;
            if (w > ext_w) ext_w = w;
            if (h > ext_h) ext_h = h;
        }
    }
    L.ext_w = ext_w;
    L.ext_h = ext_h;
    const bool vec = (p->out_w % 4 == 0) && (((uintptr_t)p->out & 15) == 0) && p->color_op != RB200_COLOR_BLEND;
    dim3 grid;
    int threads;
    L.pitch = 0;
    size_t smem = 0;
    if (vec) {
        // a tile = th full source rows staged in shared memory (up to 24 KB), about 8 four-pixel items per thread
        int pitch = (15 + ext_w * 3 + 16 + 15) & ~15;
        int gpr = (ext_w + 3) / 4;
        int th = (8 * 256 + gpr - 1) / gpr;
        if (th * pitch > 24 * 1024) th = 24 * 1024 / pitch;
        if (th < 1) th = 1;
        if (th > ext_h) th = ext_h;
        // keep at least ~4 CTAs per SM in flight for small batches
        while (th > 1 && (long)n * ((ext_h + th - 1) / th) < 4 * 148) th = (th + 1) / 2;
        L.th = th;
        L.pitch = pitch;
        L.tiles_x = 1;
        threads = 256;
        grid = dim3((unsigned)((ext_h + th - 1) / th), (unsigned)n);
        smem = 16 + 1024 + (size_t)th * pitch;
        if (smem > 200 * 1024) {
            set_error("rb200k_pointwise: rows of %d pixels are too wide", ext_w);
            return RB200_E_LIMIT;
        }
    } else {
        int tiles_x = (ext_w + 255) / 256;
        threads = ((ext_w + tiles_x - 1) / tiles_x + 31) & ~31;
        L.tiles_x = (ext_w + threads - 1) / threads;
        L.th = 8;
        int tiles_y = (ext_h + L.th - 1) / L.th;
        grid = dim3((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
    }

    // the fast arithmetic exists for ColorTwist (Hue / Saturation are the same operator) on the uint8 vector kernel
    // without normalisation or channel reversal; everything else runs the exact code
    const int op = (p->color_op == RB200_COLOR_TWIST && p->arith == RB200_ARITH_FAST && vec && p->out_dtype == RB200_UINT8 &&
                    !p->normalize && !p->reverse_channels) ? kColorTwistFast : p->color_op;
#define RB200_DISPATCH(T, LAY) return launch_color<T, LAY>(op, vec, grid, threads, smem, stream, arena, samples, L)
    if (p->out_layout == RB200_NCHW) {
        if (p->out_dtype == RB200_FP32) RB200_DISPATCH(float, RB200_NCHW);
        if (p->out_dtype == RB200_FP16) RB200_DISPATCH(__half, RB200_NCHW);
        RB200_DISPATCH(uint8_t, RB200_NCHW);
    } else {
        if (p->out_dtype == RB200_FP32) RB200_DISPATCH(float, RB200_NHWC);
        if (p->out_dtype == RB200_FP16) RB200_DISPATCH(__half, RB200_NHWC);
        RB200_DISPATCH(uint8_t, RB200_NHWC);
    }
#undef RB200_DISPATCH
}

extern "C" int rb200k_pointwise(const uint8_t* arena, const rb200_pointwise_sample* samples,
                                const rb200_pointwise_sample* h_samples, int n, const rb200_pointwise_params* p,
                                void* stream_v) {
    return pointwise_launch(arena, samples, h_samples, n, p, stream_v, kDefaultWaitCycles, -1);
}

extern "C" int rb200k_pointwise_probe(const uint8_t* arena, const rb200_pointwise_sample* samples,
                                      const rb200_pointwise_sample* h_samples, int n, const rb200_pointwise_params* p,
                                      void* stream_v, uint64_t wait_cycles, int skip_row) {
    return pointwise_launch(arena, samples, h_samples, n, p, stream_v, wait_cycles, skip_row);
}
