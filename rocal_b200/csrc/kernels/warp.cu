// Affine gather (WarpAffine / Rotate): uint8 HWC -> uint8 HWC, bilinear, constant-zero border.
//
// grid = (32 x 32 output tiles, samples), 256 threads, four pixels per thread. A CTA maps the four
// corners of its tile through the sample's 2x3 table, stages the bounding box of the source
// footprint (clamped to the image, one 1-D bulk copy per source row completing on an mbarrier) in
// shared memory and interpolates from there; a footprint that does not fit the shared-memory budget
// (strong minification) is gathered from global memory instead. Waits are bounded: on a time-out the
// kernel raises g_warp_timeout and returns.
//
// Coordinates: dx = x - (dst_w/2), dy = y - (dst_h/2) (integer halves);
//   sx = fma(m00, dx, fma(m01, dy, t0 + src_w/2)),  sy = fma(m10, dx, fma(m11, dy, t1 + src_h/2)).
// A position whose floor lies outside [0, src-1] gives 0; otherwise both taps are clamped to
// [0, src-2] and blended with the fmaf nest of the bilinear helper in
// rocAL/rocAL_hip/rocal_hip_kernels.cpp:332-343,388-409.
#include "common.cuh"

namespace rb200 {

constexpr int kWarpTile = 32;
constexpr int kWarpStageBytes = 20 * 1024;   // enough for a 32x32 tile rotated by 45 degrees at scale 0.8

struct WarpLaunch {
    uint8_t* out;
    int out_w, out_h;
    int tiles_x;
    int fill_padding;
    uint32_t magic;     // 0x4B000000
};

__device__ int g_warp_timeout = 0;

__device__ __forceinline__ uint32_t wp_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wp_mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool wp_mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (wp_mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < (1 << 24); i++) {
        if (wp_mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > 2000000000LL) break;
    }
    return false;
}

struct WarpMap {
    float m0, m1, m2, m3, t0, t1, cx, cy;
};

__device__ __forceinline__ void warp_source(const WarpMap& M, int x, int y, float& sx, float& sy) {
    const float dx = sub_rn((float)x, M.cx), dy = sub_rn((float)y, M.cy);
    sx = fmaf(M.m0, dx, fmaf(M.m1, dy, M.t0));
    sy = fmaf(M.m2, dx, fmaf(M.m3, dy, M.t1));
}

// Three bytes at any byte offset of a 4-byte aligned shared-memory block, plus the byte after them.
__device__ __forceinline__ uint32_t lds_px(const uint8_t* base, int off) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(base + (off & ~3));
    return __funnelshift_r(w[0], w[1], (uint32_t)off << 3);
}
__device__ __forceinline__ uint32_t ldg_px(const uint8_t* p) {
    return (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + 1) << 8) | ((uint32_t)__ldg(p + 2) << 16);
}

__global__ void __launch_bounds__(256) warp_affine_kernel(const uint8_t* __restrict__ arena,
                                                          const rb200_warp_sample* __restrict__ samples,
                                                          const WarpLaunch L) {
    // Layout: mbarrier (16 bytes) | staged source rows
    extern __shared__ __align__(16) uint8_t wsm[];
    __shared__ int stage_flag;
    uint8_t* stage = wsm + 16;
    const uint32_t bar = wp_smem_u32(wsm);

    const int n = blockIdx.y;
    const int tile_x0 = (blockIdx.x % L.tiles_x) * kWarpTile;
    const int tile_y0 = (blockIdx.x / L.tiles_x) * kWarpTile;
    const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;

    const rb200_warp_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    const int w = min(s.dst_w, L.out_w), h = min(s.dst_h, L.out_h);
    const int W = s.src_w, H = s.src_h;
    const bool tile_valid = tile_x0 < w && tile_y0 < h && W > 0 && H > 0;

    WarpMap M;
    M.m0 = s.m[0]; M.m1 = s.m[1]; M.m2 = s.m[2]; M.m3 = s.m[3];
    M.t0 = add_rn(s.m[4], mul_rn((float)W, 0.5f));
    M.t1 = add_rn(s.m[5], mul_rn((float)H, 0.5f));
    M.cx = (float)(s.dst_w / 2);
    M.cy = (float)(s.dst_h / 2);

    bool staged = false;
    int bx0 = 0, by0 = 0, pitch = 0;
    uint32_t base_mod = 0, stride_mod = 0;
    if (tile_valid) {
        // Bounding box of the tile's source footprint: an affine map takes its extremes at the corners.
        const int cx1 = min(tile_x0 + kWarpTile, w) - 1, cy1 = min(tile_y0 + kWarpTile, h) - 1;
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
        bx0 = min(max((int)floorf(fx_min) - 1, 0), max(W - 2, 0));
        by0 = min(max((int)floorf(fy_min) - 1, 0), max(H - 2, 0));
        int bx1 = min(max((int)floorf(fx_max) + 2, bx0), W - 1);
        int by1 = min(max((int)floorf(fy_max) + 2, by0), H - 1);
        const int rows = by1 - by0 + 1;
        const int rowbytes = (bx1 - bx0 + 1) * 3;
        pitch = (15 + rowbytes + 8 + 15) & ~15;
        staged = (long)rows * pitch <= kWarpStageBytes;
        base_mod = (uint32_t)((uintptr_t)(img + (size_t)bx0 * 3) & 15);
        stride_mod = s.src_stride & 15;
        if (staged) {
            if (threadIdx.x == 0) {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(min(rows, 32)) : "memory");
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncthreads();
            if (threadIdx.x < 32 && (int)threadIdx.x < rows) {
                uint32_t total = 0;
                for (int r = threadIdx.x; r < rows; r += 32) {
                    const uint32_t m = (base_mod + (uint32_t)(by0 + r) * stride_mod) & 15;
                    total += ((m + (uint32_t)rowbytes + 15) >> 4) << 4;
                }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
                for (int r = threadIdx.x; r < rows; r += 32) {
                    const uint8_t* g = img + (size_t)(by0 + r) * s.src_stride + (size_t)bx0 * 3;
                    const uint32_t m = (uint32_t)((uintptr_t)g & 15);
                    const uint32_t bytes = ((m + (uint32_t)rowbytes + 15) >> 4) << 4;
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(wp_smem_u32(stage + (size_t)r * pitch)), "l"(g - m), "r"(bytes), "r"(bar) : "memory");
                }
            }
            // Warp 0 waits for the copies (bounded); the other warps sleep at the barrier instead of polling.
            if (threadIdx.x < 32) {
                const bool ok = wp_mbar_wait_bounded(bar, 0);
                if (threadIdx.x == 0) {
                    stage_flag = ok ? 1 : 0;
                    if (!ok) {
                        atomicExch(&g_warp_timeout, 1);
                        wp_mbar_wait_bounded(bar, 0);   // second bounded chance for copies still in flight
                    }
                }
            }
            __syncthreads();
            if (!stage_flag) return;
        }
    }

    const int xh = max(W - 2, 0), yh = max(H - 2, 0);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const int x = tile_x0 + lx, y = tile_y0 + ly + 8 * k;
        if (x >= L.out_w || y >= L.out_h) continue;
        uint8_t* o = L.out + (((size_t)n * L.out_h + y) * L.out_w + x) * 3;
        if (x >= w || y >= h) {
            if (L.fill_padding) { o[0] = 0; o[1] = 0; o[2] = 0; }
            continue;
        }
        float sx, sy;
        warp_source(M, x, y, sx, sy);
        const float fx = floorf(sx), fy = floorf(sy);
        float v0 = 0.f, v1 = 0.f, v2 = 0.f;
        // Written so that NaN coordinates fall through to the interpolation exactly as in the checker.
        if (!(fx < 0.f || fy < 0.f || fx > (float)(W - 1) || fy > (float)(H - 1))) {
            const float wx = sub_rn(sx, fx), wy = sub_rn(sy, fy);
            const float owx = sub_rn(1.0f, wx), owy = sub_rn(1.0f, wy);
            const int x0 = (int)fminf(fmaxf(fx, 0.f), (float)xh);
            const int y0 = (int)fminf(fmaxf(fy, 0.f), (float)yh);
            const int x1 = (int)fminf(fmaxf(add_rn(fx, 1.0f), 0.f), (float)xh);
            const int y1 = (int)fminf(fmaxf(add_rn(fy, 1.0f), 0.f), (float)yh);
            uint32_t tl, tr, bl, br;
            if (staged) {
                const int r0 = y0 - by0, r1 = y1 - by0;
                const int o0 = r0 * pitch + (int)((base_mod + (uint32_t)y0 * stride_mod) & 15);
                const int o1 = r1 * pitch + (int)((base_mod + (uint32_t)y1 * stride_mod) & 15);
                const int cl = (x0 - bx0) * 3, cr = (x1 - bx0) * 3;
                tl = lds_px(stage, o0 + cl);
                tr = lds_px(stage, o0 + cr);
                bl = lds_px(stage, o1 + cl);
                br = lds_px(stage, o1 + cr);
            } else {
                const uint8_t* p0 = img + (size_t)y0 * s.src_stride;
                const uint8_t* p1 = img + (size_t)y1 * s.src_stride;
                tl = ldg_px(p0 + x0 * 3);
                tr = ldg_px(p0 + x1 * 3);
                bl = ldg_px(p1 + x0 * 3);
                br = ldg_px(p1 + x1 * 3);
            }
            const float w00 = mul_rn(owy, owx), w01 = mul_rn(owy, wx), w10 = mul_rn(wy, owx);
            float v[3];
#pragma unroll
            for (int c = 0; c < 3; c++) {
                const uint32_t sel = 0x7650u + c;
                const float ftl = sub_rn(__uint_as_float(__byte_perm(tl, L.magic, sel)), 8388608.0f);
                const float ftr = sub_rn(__uint_as_float(__byte_perm(tr, L.magic, sel)), 8388608.0f);
                const float fbl = sub_rn(__uint_as_float(__byte_perm(bl, L.magic, sel)), 8388608.0f);
                const float fbr = sub_rn(__uint_as_float(__byte_perm(br, L.magic, sel)), 8388608.0f);
                float acc = mul_rn(mul_rn(fbr, wy), wx);
                acc = fmaf(fbl, w10, acc);
                acc = fmaf(ftr, w01, acc);
                acc = fmaf(ftl, w00, acc);
                v[c] = sat_round_u8f(acc);
            }
            v0 = v[0]; v1 = v[1]; v2 = v[2];
        }
        o[0] = (uint8_t)v0;
        o[1] = (uint8_t)v1;
        o[2] = (uint8_t)v2;
    }
}

int warp_timeout_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_warp_timeout, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_warp_timeout, &zero, sizeof(int));
    return v;
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
    L.tiles_x = (p->out_w + kWarpTile - 1) / kWarpTile;
    int tiles_y = (p->out_h + kWarpTile - 1) / kWarpTile;
    dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
    warp_affine_kernel<<<grid, 256, 16 + kWarpStageBytes, (cudaStream_t)stream_v>>>(arena, samples, L);
    RB200_CHECK_LAUNCH("warp_affine_kernel");
    return RB200_OK;
}
