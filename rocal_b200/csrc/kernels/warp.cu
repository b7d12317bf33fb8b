// Affine gather (WarpAffine / Rotate): uint8 HWC -> uint8 HWC, bilinear, constant-zero border.
//
// grid = (64 x 32 output tiles, samples), 256 threads, eight consecutive pixels of a row per thread. A CTA maps the four
// corners of its tile through the sample's 2x3 table, stages the bounding box of the source
// footprint (clamped to the image) in shared memory with 16-byte asynchronous copies and interpolates
// from there; a footprint that does not fit the shared-memory budget (strong minification) is gathered
// from global memory instead. The staged rows are short (about 130 bytes at scale 1), which is why
// they are fetched as per-thread 16-byte copies: one bulk copy per row costs more issue slots than the
// row is worth.
//
// Coordinates: dx = x - (dst_w/2), dy = y - (dst_h/2) (integer halves);
//   sx = fma(m00, dx, fma(m01, dy, t0 + src_w/2)),  sy = fma(m10, dx, fma(m11, dy, t1 + src_h/2)).
// A position whose floor lies outside [0, src-1] gives 0; otherwise both taps are clamped to
// [0, src-2] and blended with the fmaf nest of the bilinear helper in
// rocAL/rocAL_hip/rocal_hip_kernels.cpp:332-343,388-409.
#include "common.cuh"

namespace rb200 {

constexpr int kWarpTileW = 64, kWarpTileH = 32;
constexpr int kWarpPx = 8;                   // consecutive pixels of a row per thread: 8 threads span the tile
constexpr int kWarpStageBytes = 32 * 1024;   // enough for a 64x32 tile rotated by 45 degrees at scale 0.8

struct WarpLaunch {
    uint8_t* out;
    int out_w, out_h;
    int tiles_x;
    int fill_padding;
    uint32_t magic;     // 0x4B000000
    int vec_store;      // rows of the output start on 4-byte boundaries
    int overlap;        // 1 = independent of the preceding kernel, wait for it only before exit
    int* status;        // bounds-checking build: written with 2 when a sample's source leaves the arena
    ArenaBounds bounds; // bounds-checking build: the addresses the launch may read
};

struct WarpMap {
    float m0, m1, m2, m3, t0, t1, cx, cy;
};

__device__ __forceinline__ void warp_source(const WarpMap& M, int x, int y, float& sx, float& sy) {
    const float dx = sub_rn((float)x, M.cx), dy = sub_rn((float)y, M.cy);
    sx = fmaf(M.m0, dx, fmaf(M.m1, dy, M.t0));
    sy = fmaf(M.m2, dx, fmaf(M.m3, dy, M.t1));
}

// Six bytes (two neighbouring pixels) at any byte offset of a 4-byte aligned shared-memory block:
// P = bytes 0..3, Q = bytes 4..7.
__device__ __forceinline__ void lds_pair(const uint8_t* base, int off, uint32_t& P, uint32_t& Q) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(base + (off & ~3));
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    const uint32_t sh = (uint32_t)off << 3;
    P = __funnelshift_r(w0, w1, sh);
    Q = __funnelshift_r(w1, w2, sh);
}
__device__ __forceinline__ uint32_t ldg_px(const uint8_t* p) {
    return (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + 1) << 8) | ((uint32_t)__ldg(p + 2) << 16);
}

// One pixel's four taps, each with its three channels in bytes 0..2 (top row t*, bottom row b*).
struct WarpTaps {
    uint32_t tL, tR, bL, bR;
};

// Blend of two pixels at once: every float operation is a packed f32x2 instruction (one rounding per
// lane, so each lane equals the scalar sequence). The 2^23 exponent trick turns a byte into a float with
// one permute and one subtraction. Returns, per pixel, the three rounded channels in bytes 0..2 (byte 3
// is unspecified).
__device__ __forceinline__ uint2 blend_px2(const WarpTaps& A, const WarpTaps& B, float2 wx, float2 wy, uint32_t magic) {
    const float2 nk23 = make_float2(-8388608.0f, -8388608.0f), kround = make_float2(12582912.0f, 12582912.0f);
    const float2 owx = make_float2(sub_rn(1.0f, wx.x), sub_rn(1.0f, wx.y));
    const float2 owy = make_float2(sub_rn(1.0f, wy.x), sub_rn(1.0f, wy.y));
    const float2 w00 = mul2(owy, owx), w01 = mul2(owy, wx), w10 = mul2(wy, owx);
    uint32_t ua[3], ub[3];
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const uint32_t sel = 0x7650u + c;
        float2 ftl, fbl, ftr, fbr;
        ftl.x = __uint_as_float(__byte_perm(A.tL, magic, sel));
        ftl.y = __uint_as_float(__byte_perm(B.tL, magic, sel));
        fbl.x = __uint_as_float(__byte_perm(A.bL, magic, sel));
        fbl.y = __uint_as_float(__byte_perm(B.bL, magic, sel));
        ftr.x = __uint_as_float(__byte_perm(A.tR, magic, sel));
        ftr.y = __uint_as_float(__byte_perm(B.tR, magic, sel));
        fbr.x = __uint_as_float(__byte_perm(A.bR, magic, sel));
        fbr.y = __uint_as_float(__byte_perm(B.bR, magic, sel));
        ftl = add2(ftl, nk23);
        fbl = add2(fbl, nk23);
        ftr = add2(ftr, nk23);
        fbr = add2(fbr, nk23);
        float2 acc = mul2(mul2(fbr, wy), wx);
        acc = fma2(fbl, w10, acc);
        acc = fma2(ftr, w01, acc);
        acc = fma2(ftl, w00, acc);
        // 0 <= acc < 255.5 (a convex blend of bytes up to rounding): adding 1.5 * 2^23 leaves the
        // nearest-even integer in the low byte, which is the saturating conversion of the checker.
        acc = add2(acc, kround);
        ua[c] = __float_as_uint(acc.x);
        ub[c] = __float_as_uint(acc.y);
    }
    uint2 r;
    r.x = __byte_perm(__byte_perm(ua[0], ua[1], 0x0040u), ua[2], 0x4410u);
    r.y = __byte_perm(__byte_perm(ub[0], ub[1], 0x0040u), ub[2], 0x4410u);
    return r;
}

// What warp 0 works out for the CTA: the staged box of the source and its shared-memory geometry.
struct WarpHeader {
    int staged, bx0, by0, bx1, by1, pitch;
};

// One thread's run of kWarpPx consecutive output pixels, two at a time. [xlo,xhi] x [ylo,yhi] is the
// range of tap positions that may be read (the staged box, or the image); in-range pixels never leave
// it, the clamps only keep the loads of out-of-range lanes harmless. A pixel pair is skipped when no
// lane of the warp has a source position inside the image (the zero border of a rotated frame),
// otherwise computed without branches and zeroed by a select.
template <bool STAGED>
__device__ __forceinline__ void warp_taps(WarpTaps& T, int ix, int iy, int xlo, int xhi, int ylo, int yhi, int xh, int yh,
                                          const uint8_t* __restrict__ img, uint32_t src_stride, const uint8_t* stage,
                                          int tab_off) {
    const int x0 = min(max(ix, xlo), xhi);
    const int yc = min(max(iy, ylo), yhi);
    if (STAGED) {
        const int2 ro = *reinterpret_cast<const int2*>(stage + tab_off + yc * 8);
        uint32_t tP, tQ, bP, bQ;
        lds_pair(stage, ro.x + x0 * 3, tP, tQ);
        lds_pair(stage, ro.y + x0 * 3, bP, bQ);
        // The right tap is the next pixel (bytes 3..5 of the six), except in the last two columns, where
        // it is clamped onto the left one.
        const uint32_t rsel = ix >= xh ? 0x3210u : 0x0543u;
        T.tL = tP;
        T.bL = bP;
        T.tR = __byte_perm(tP, tQ, rsel);
        T.bR = __byte_perm(bP, bQ, rsel);
    } else {
        const uint8_t* p0 = img + (size_t)min(yc, yh) * src_stride + x0 * 3;
        const uint8_t* p1 = img + (size_t)min(yc + 1, yh) * src_stride + x0 * 3;
        const int step = x0 < xh ? 3 : 0;   // right tap clamped onto the left one in the last two columns
        T.tL = ldg_px(p0);
        T.bL = ldg_px(p1);
        T.tR = ldg_px(p0 + step);
        T.bR = ldg_px(p1 + step);
    }
}

template <bool STAGED>
__device__ __forceinline__ void warp_pixels(uint32_t (&px)[kWarpPx], const WarpMap& M, const uint8_t* __restrict__ img,
                                            uint32_t src_stride, int W, int H, int x, int y, int wlim, int xlo,
                                            int xhi, int ylo, int yhi, const uint8_t* stage, int tab_off,
                                            uint32_t magic) {
    const int xh = max(W - 2, 0), yh = max(H - 2, 0);
    const float dy = sub_rn((float)y, M.cy);
    const float rx = fmaf(M.m1, dy, M.t0), ry = fmaf(M.m3, dy, M.t1);
    const float dx0 = sub_rn((float)x, M.cx);
    const float Wf = (float)W, Hf = (float)H;
#pragma unroll
    for (int k = 0; k < kWarpPx; k += 2) {
        const float dxa = add_rn(dx0, (float)k), dxb = add_rn(dx0, (float)(k + 1));     // exact: small integers
        const float sxa = fmaf(M.m0, dxa, rx), sya = fmaf(M.m2, dxa, ry);
        const float sxb = fmaf(M.m0, dxb, rx), syb = fmaf(M.m2, dxb, ry);
        // floor(s) in [0, size-1]  <=>  0 <= s < size; NaN fails and gives 0 like the checker's clamps
        const bool oka = x + k < wlim && sxa >= 0.f && sxa < Wf && sya >= 0.f && sya < Hf;
        const bool okb = x + k + 1 < wlim && sxb >= 0.f && sxb < Wf && syb >= 0.f && syb < Hf;
        px[k] = 0u;
        px[k + 1] = 0u;
        if (__any_sync(0xffffffffu, oka || okb)) {
            const int ixa = __float2int_rd(sxa), iya = __float2int_rd(sya);
            const int ixb = __float2int_rd(sxb), iyb = __float2int_rd(syb);
            const float2 wx = make_float2(sub_rn(sxa, (float)ixa), sub_rn(sxb, (float)ixb));
            const float2 wy = make_float2(sub_rn(sya, (float)iya), sub_rn(syb, (float)iyb));
            WarpTaps A, B;
            warp_taps<STAGED>(A, ixa, iya, xlo, xhi, ylo, yhi, xh, yh, img, src_stride, stage, tab_off);
            warp_taps<STAGED>(B, ixb, iyb, xlo, xhi, ylo, yhi, xh, yh, img, src_stride, stage, tab_off);
            const uint2 v = blend_px2(A, B, wx, wy, magic);
            px[k] = oka ? v.x : 0u;
            px[k + 1] = okb ? v.y : 0u;
        }
    }
}

__device__ __forceinline__ void warp_affine_tile(const uint8_t* __restrict__ arena, const rb200_warp_sample* __restrict__ samples,
                                                 const WarpLaunch& L, uint8_t* stage, WarpHeader& hdr) {

    const int n = blockIdx.y;
    const int tile_x0 = (blockIdx.x % L.tiles_x) * kWarpTileW;
    const int tile_y0 = (blockIdx.x / L.tiles_x) * kWarpTileH;
    const int x = tile_x0 + kWarpPx * (threadIdx.x & 7), y = tile_y0 + (threadIdx.x >> 3);

    const rb200_warp_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    const int w = min(s.dst_w, L.out_w), h = min(s.dst_h, L.out_h);
    const int W = s.src_w, H = s.src_h;
    // (bounds-checking build) a sample whose source image leaves the arena is reported and treated as empty
    const bool tile_valid = tile_x0 < w && tile_y0 < h && W > 0 && H > 0 &&
                            rect_in_bounds(L.bounds, img, s.src_stride, 0, 0, W, H, L.status);
    if (!tile_valid && !L.fill_padding) return;

    WarpMap M;
    M.m0 = s.m[0]; M.m1 = s.m[1]; M.m2 = s.m[2]; M.m3 = s.m[3];
    M.t0 = add_rn(s.m[4], mul_rn((float)W, 0.5f));
    M.t1 = add_rn(s.m[5], mul_rn((float)H, 0.5f));
    M.cx = (float)(s.dst_w / 2);
    M.cy = (float)(s.dst_h / 2);

    uint32_t px[kWarpPx];
#pragma unroll
    for (int k = 0; k < kWarpPx; k++) px[k] = 0u;
    if (tile_valid) {
        const int xh = max(W - 2, 0), yh = max(H - 2, 0);
        if (threadIdx.x < 32) {
            // Bounding box of the tile's source footprint: an affine map takes its extremes at the corners.
            const int cx1 = min(tile_x0 + kWarpTileW, w) - 1, cy1 = min(tile_y0 + kWarpTileH, h) - 1;
            float ax, ay, bx, by, cx, cy, dx, dy;
            warp_source(M, tile_x0, tile_y0, ax, ay);
            warp_source(M, cx1, tile_y0, bx, by);
            warp_source(M, tile_x0, cy1, cx, cy);
            warp_source(M, cx1, cy1, dx, dy);
            const float lim = 1.0e6f;
            const float fx_min = fminf(fmaxf(fminf(fminf(ax, bx), fminf(cx, dx)), -lim), lim);
            const float fx_max = fminf(fmaxf(fmaxf(fmaxf(ax, bx), fmaxf(cx, dx)), -lim), lim);
            const float fy_min = fminf(fmaxf(fminf(fminf(ay, by), fminf(cy, dy)), -lim), lim);
            const float fy_max = fminf(fmaxf(fmaxf(fmaxf(ay, by), fmaxf(cy, dy)), -lim), lim);
            // one pixel of margin each side, then clamp so that the box holds every clamped tap
            WarpHeader hh;
            hh.bx0 = min(max((int)floorf(fx_min) - 1, 0), xh);
            hh.by0 = min(max((int)floorf(fy_min) - 1, 0), yh);
            hh.bx1 = min(max((int)floorf(fx_max) + 2, hh.bx0), W - 1);
            hh.by1 = min(max((int)floorf(fy_max) + 2, hh.by0), H - 1);
            const int rows = hh.by1 - hh.by0 + 1;
            hh.pitch = (15 + (hh.bx1 - hh.bx0 + 1) * 3 + 12 + 15) & ~15;
            hh.staged = (long)rows * (hh.pitch + 8) <= kWarpStageBytes;
            if (threadIdx.x == 0) hdr = hh;
        }
        __syncthreads();
        const WarpHeader hh = hdr;
        // the thread's row and first column; threads outside the sample (or the canvas) compute nothing
        const int wlim = (y < h) ? w : 0;
        if (hh.staged) {
            // 16 rows per pass, 16 lanes per row, 16-byte chunks from the aligned-down start of each row.
            // Entry r of the table serves floor(sy) = by0 + r: byte offsets (of source column 0, from the
            // stage base) of the two tap rows min(iy, H-2) and min(iy+1, H-2).
            const int rows = hh.by1 - hh.by0 + 1, rowbytes = (hh.bx1 - hh.bx0 + 1) * 3;
            int2* tab = reinterpret_cast<int2*>(stage + (size_t)rows * hh.pitch);
            const uint32_t base_mod = (uint32_t)((uintptr_t)(img + (size_t)hh.bx0 * 3) & 15);
            const uint32_t stride_mod = s.src_stride & 15;
            for (int r = threadIdx.x; r < rows; r += 256) {
                const int iy = hh.by0 + r;
                const int ya = min(iy, yh), yb = min(iy + 1, yh);
                int2 e;
                e.x = (ya - hh.by0) * hh.pitch + (int)((base_mod + (uint32_t)ya * stride_mod) & 15) - hh.bx0 * 3;
                e.y = (yb - hh.by0) * hh.pitch + (int)((base_mod + (uint32_t)yb * stride_mod) & 15) - hh.bx0 * 3;
                tab[r] = e;
            }
            const int c0 = (threadIdx.x & 15) * 16, r0 = threadIdx.x >> 4;
            const uint8_t* g = img + (size_t)(hh.by0 + r0) * s.src_stride + (size_t)hh.bx0 * 3 + c0;
            uint32_t d = (uint32_t)__cvta_generic_to_shared(stage) + (uint32_t)(r0 * hh.pitch + c0);
            const size_t gstep = (size_t)16 * s.src_stride;
            const uint32_t dstep = 16u * (uint32_t)hh.pitch;
            for (int r = r0; r < rows; r += 16, g += gstep, d += dstep) {
                const int m = (int)((uintptr_t)g & 15);
                for (int c = c0; c < m + rowbytes; c += 256)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d + (uint32_t)(c - c0)), "l"(g - m + (c - c0)) : "memory");
            }
            cp_async_commit_wait_all();
            __syncthreads();
            warp_pixels<true>(px, M, img, s.src_stride, W, H, x, y, wlim, hh.bx0, min(hh.bx1, xh), hh.by0, hh.by1,
                              stage, (rows * hh.pitch) - hh.by0 * 8, L.magic);
        } else {
            warp_pixels<false>(px, M, img, s.src_stride, W, H, x, y, wlim, 0, xh, 0, H - 1, stage, 0, L.magic);
        }
    }

    if (x >= L.out_w || y >= L.out_h) return;
    const int lim = (tile_valid && y < h) ? w : 0;        // pixels at or beyond lim are padding
    if (x >= lim && !L.fill_padding) return;
    uint8_t* o = L.out + (((size_t)n * L.out_h + y) * L.out_w + x) * 3;
#pragma unroll
    for (int g = 0; g < kWarpPx; g += 4) {
        if (L.vec_store && (x + g + 3 < lim || (L.fill_padding && x + g + 3 < L.out_w))) {
            uint32_t* o4 = reinterpret_cast<uint32_t*>(o + 3 * g);
            o4[0] = __byte_perm(px[g + 0], px[g + 1], 0x4210u);
            o4[1] = __byte_perm(px[g + 1], px[g + 2], 0x5421u);
            o4[2] = __byte_perm(px[g + 2], px[g + 3], 0x6542u);
        } else {
#pragma unroll
            for (int k = g; k < g + 4; k++) {
                if (x + k >= L.out_w) break;
                if (x + k >= lim && !L.fill_padding) continue;
                o[3 * k + 0] = (uint8_t)(px[k]);
                o[3 * k + 1] = (uint8_t)(px[k] >> 8);
                o[3 * k + 2] = (uint8_t)(px[k] >> 16);
            }
        }
    }
}

__global__ void __launch_bounds__(256, 5) warp_affine_kernel(const uint8_t* __restrict__ arena,
                                                          const rb200_warp_sample* __restrict__ samples,
                                                          const WarpLaunch L) {
    // Layout: staged source rows | per-row offset pairs
    extern __shared__ __align__(16) uint8_t stage[];
    __shared__ WarpHeader hdr;
    pdl_launch_dependents();
    if (!L.overlap) pdl_wait();
    warp_affine_tile(arena, samples, L, stage, hdr);
    if (L.overlap) pdl_wait();      // completion of this launch implies completion of the kernel before it
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_warp_affine(const uint8_t* arena, const rb200_warp_sample* samples, int n,
                                  const rb200_warp_params* p, void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_warp_affine: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_warp_affine: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    WarpLaunch L;
    L.out = (uint8_t*)p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.fill_padding = p->fill_padding;
    L.magic = 0x4B000000u;
    L.vec_store = (p->out_w % 4 == 0) && (((uintptr_t)p->out & 3) == 0);
    L.overlap = p->overlap ? 1 : 0;
    L.status = p->status ? p->status : default_status_word();
    if (!L.status) {
        set_error("rb200k_warp_affine: the device's status word cannot be addressed");
        return RB200_E_CUDA;
    }
    L.bounds = arena_bounds(arena, p->arena_bytes);
    if (p->out_bytes && (uint64_t)n * p->out_w * p->out_h * 3 > p->out_bytes) {
        set_error("rb200k_warp_affine: %d samples of %d x %d x 3 bytes do not fit the %llu-byte output", n, p->out_w, p->out_h,
                  (unsigned long long)p->out_bytes);
        return RB200_E_INVALID;
    }
    L.tiles_x = (p->out_w + kWarpTileW - 1) / kWarpTileW;
    int tiles_y = (p->out_h + kWarpTileH - 1) / kWarpTileH;
    dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
    launch_overlapped(warp_affine_kernel, grid, dim3(256), (size_t)kWarpStageBytes, (cudaStream_t)stream_v, arena, samples, L);
    RB200_CHECK_LAUNCH("warp_affine_kernel");
    return RB200_OK;
}
