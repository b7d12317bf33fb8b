// Bilinear resample family: [crop ->] resize [-> crop] [-> mirror] [-> normalize] in one pass.
//
// One launch covers the whole ragged batch: grid = (tiles of the output extent, samples).
//
// Staged kernel (the fast path). A CTA owns an output tile of TH rows. It stages the source rows
// its taps touch into shared memory with 16-byte cp.async copies (global addresses rounded down
// to 16 bytes, so every copy is aligned whatever the row pitch of the packed uint8 HWC source;
// one warp per source row), then every thread interpolates TWO horizontally adjacent output
// pixels per row from shared memory:
//   * a tap pair (x0, x0+1) is 6 contiguous bytes: three 32-bit shared loads + two funnel shifts;
//   * uint8 -> float by PRMT into the mantissa of 2^23 and one subtraction (no conversion unit);
//   * all float math on the two pixels runs as Blackwell packed f32x2 instructions
//     (mul/add/fma.rn.f32x2: one rounding per lane, so results equal the scalar sequence);
//   * the pixel pair leaves as one half2 / float2 store per channel plane.
// Column-dependent values (tap offsets, x weights) are computed once per thread and reused for
// all rows of the tile.
//
// Direct kernel: same arithmetic, taps read straight from global memory; used when the caller
// gives no host copy of the table (the launch cannot be sized for staging) or a tile's source
// span does not fit in shared memory.
//
// The interpolation follows the reference's HIP bilinear kernel
// (rocAL/rocAL_hip/rocal_hip_kernels.cpp:311-343, 388-409, 425-430): source location
// dst*ratio + (ratio-1)/2 + roi.x, floor, taps clamped to [roi.x, roi.x2-1], the fmaf nest
// TL*(1-wy)(1-wx) + (TR*(1-wy)wx + (BL*wy(1-wx) + BR*wy*wx)), round-to-nearest-even uint8.
#include <cstdlib>

#include <mutex>
#include <vector>

#include <type_traits>

#include "common.cuh"

namespace rb200 {

struct ResampleLaunch {
    void* out;
    int out_w, out_h;
    int ext_w, ext_h;   // extent covered by the grid
    int tiles_x;
    int th;             // rows per tile
    int pitch;          // bytes per staged row (multiple of 16)
    int twh;            // staged kernel: threads per row group (each owns two columns)
    int groups;         // staged kernel: row groups per CTA
    int strip_rows;     // stream kernel: output rows per CTA
    int ns, ns_log2;    // stream kernel: ring stages (power of two)
    int pair_ok;        // paired (2-element) stores are aligned
    int normalize, fill_padding;
    int filter;         // generic-filter kernel: RB200_INTERP_* (triangular, bicubic, lanczos, gaussian, nearest)
    float mul[3], add[3];
    uint32_t magic;     // 0x4B000000 (bits of 2^23), passed as a parameter so that PRMT reads it
                        // from the constant bank instead of a re-materialised register
    int* status;        // stream kernel: written with 1 when a bounded wait gives up
    long long wait_cycles;   // stream kernel: limit of every mbarrier wait, SM clock cycles
    int skip_row;       // stream kernel, self-test: the producer issues no copy from this strip row on (-1: all)
    int overlap;        // stream kernel: 1 = independent of the preceding kernel, wait for it only before exit
    int row_ring;       // stream kernel: 1 = ring of distinct source rows (host-memory sources), 0 = ring of tap-row pairs
    ArenaBounds bounds; // bounds-checking build: the addresses the launch may read
};

struct RowInfo {
    float wy, owy;
    int off0, off1;     // staged: byte offset of the row's first staged pixel in shared memory
                        // direct: source row index of the two taps
};

__device__ __forceinline__ float src_location(int d, float ratio, float offset, int roi_start) {
    return add_rn(fmaf((float)d, ratio, offset), (float)roi_start);
}

__device__ __forceinline__ void clamp_taps(float f, int lo, int hi, int& t0, int& t1) {
    t0 = (int)fminf(fmaxf(f, (float)lo), (float)hi);
    t1 = (int)fminf(fmaxf(add_rn(f, 1.0f), (float)lo), (float)hi);
}

template <typename OutT, int LAYOUT>
__device__ __forceinline__ size_t out_index(int out_w, int out_h, int n, int c, int y, int x) {
    if (LAYOUT == RB200_NCHW) return (((size_t)n * 3 + c) * out_h + y) * out_w + x;
    return (((size_t)n * out_h + y) * out_w + x) * 3 + c;
}

template <typename OutT, int LAYOUT>
__device__ __forceinline__ void store3(OutT* out, int out_w, int out_h, int n, int y, int x, float v0, float v1, float v2) {
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

// Byte `sel & 7` of (w, magic = 0x4B000000) placed in the mantissa of 2^23: the float 8388608 + byte.
__device__ __forceinline__ float byte_magic(uint32_t w, uint32_t magic, uint32_t sel) {
    return __uint_as_float(__byte_perm(w, magic, sel));
}

// One column's taps of one source row: words L (bytes b..b+3) and R (bytes b+4..b+7).
__device__ __forceinline__ void fetch_pair(const uint8_t* stage, int b, uint32_t& l, uint32_t& r) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(stage + (b & ~3));
    uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    uint32_t sh = (uint32_t)b << 3;
    l = __funnelshift_r(w0, w1, sh);
    r = __funnelshift_r(w1, w2, sh);
}

struct ColumnTaps {
    int o_left;              // byte offset of the left tap from the first staged pixel
    uint32_t sel_r, sel_g, sel_b;   // PRMT selectors of the right tap's channels
    bool same;               // right tap == left tap (clamped at a border)
};

template <typename OutT>
struct PairStore;
template <>
struct PairStore<float> {
    static __device__ __forceinline__ void st(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <>
struct PairStore<__half> {
    static __device__ __forceinline__ void st(__half* p, float2 v) {
        *reinterpret_cast<__half2*>(p) = __floats2half2_rn(v.x, v.y);
    }
};
template <>
struct PairStore<uint8_t> {
    static __device__ __forceinline__ void st(uint8_t* p, float2 v) {
        uint32_t a = (uint32_t)sat_round_u8f(v.x), b = (uint32_t)sat_round_u8f(v.y);
        *reinterpret_cast<uint16_t*>(p) = (uint16_t)(a | (b << 8));
    }
};

// Per-tile values every thread needs, computed once by one thread.
struct TileHeader {
    float ratio_w, off_w;
    int x_first, nbytes;     // first staged source column, bytes staged per row
    int nslots;              // staged source rows
    int pad[3];
};

// Row table entry of the staged kernel (32 bytes: one 16-byte and one 8-byte shared load).
struct StagedRow {
    float2 wy2, owy2;        // y weights, duplicated for the packed lanes
    int off0, off1;          // byte offset of the first staged pixel of the two tap rows
    int pad[2];
};

// One output row of one thread: two adjacent pixels, three channels, blended from staged rows at byte
// offsets off0 / off1 (the row's first staged pixel) and stored at po.
// EDGE = false promises that no lane's right tap is clamped onto its left one (ct[p].same is false for both
// columns), which drops the four selects that serve those border lanes.
template <typename OutT, int LAYOUT, bool NORMALIZE, bool PAIRED, bool EDGE = true>
__device__ __forceinline__ void blend_store(const uint8_t* stage, int off0, int off1, float2 wy2, float2 owy2,
                                            const ColumnTaps (&ct)[2], float2 wx2, float2 owx2, bool second,
                                            const float (&mulv)[3], const float (&addv)[3], const uint32_t magic,
                                            OutT* po, size_t plane) {
    const float2 neg_magic = make_float2(-8388608.0f, -8388608.0f);
    const float2 rnd = make_float2(12582912.0f, 12582912.0f);
    const float2 neg_rnd = make_float2(-12582912.0f, -12582912.0f);
    uint32_t l0[2], r0[2], l1[2], r1[2];
#pragma unroll
    for (int p = 0; p < 2; p++) {
        fetch_pair(stage, off0 + ct[p].o_left, l0[p], r0[p]);
        fetch_pair(stage, off1 + ct[p].o_left, l1[p], r1[p]);
        if (EDGE) {
            r0[p] = ct[p].same ? l0[p] : r0[p];
            r1[p] = ct[p].same ? l1[p] : r1[p];
        }
    }
    const float2 w00 = mul2(owy2, owx2), w01 = mul2(owy2, wx2), w10 = mul2(wy2, owx2);
    float2 v[3];
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const uint32_t sel_l = 0x7650u + c;
        float2 tl = make_float2(byte_magic(l0[0], magic, sel_l), byte_magic(l0[1], magic, sel_l));
        float2 bl = make_float2(byte_magic(l1[0], magic, sel_l), byte_magic(l1[1], magic, sel_l));
        float2 tr, br;
        // right tap: its red byte sits in the left word unless the taps coincide
        if (c == 0) {
            tr = make_float2(byte_magic(l0[0], magic, ct[0].sel_r), byte_magic(l0[1], magic, ct[1].sel_r));
            br = make_float2(byte_magic(l1[0], magic, ct[0].sel_r), byte_magic(l1[1], magic, ct[1].sel_r));
        } else if (c == 1) {
            tr = make_float2(byte_magic(r0[0], magic, ct[0].sel_g), byte_magic(r0[1], magic, ct[1].sel_g));
            br = make_float2(byte_magic(r1[0], magic, ct[0].sel_g), byte_magic(r1[1], magic, ct[1].sel_g));
        } else {
            tr = make_float2(byte_magic(r0[0], magic, ct[0].sel_b), byte_magic(r0[1], magic, ct[1].sel_b));
            br = make_float2(byte_magic(r1[0], magic, ct[0].sel_b), byte_magic(r1[1], magic, ct[1].sel_b));
        }
        tl = add2(tl, neg_magic);
        tr = add2(tr, neg_magic);
        bl = add2(bl, neg_magic);
        br = add2(br, neg_magic);
        float2 acc = mul2(mul2(br, wy2), wx2);
        acc = fma2(bl, w10, acc);
        acc = fma2(tr, w01, acc);
        acc = fma2(tl, w00, acc);
        // The blend of uint8 values with weights in [0,1] stays inside [0,255] up to
        // rounding, so rounding to nearest even is all the uint8 quantisation needs.
        acc = add2(add2(acc, rnd), neg_rnd);
        v[c] = NORMALIZE ? fma2(acc, make_float2(mulv[c], mulv[c]), make_float2(addv[c], addv[c])) : acc;
    }
    if (PAIRED) {
        if (LAYOUT == RB200_NCHW) {
            PairStore<OutT>::st(po, v[0]);
            PairStore<OutT>::st(po + plane, v[1]);
            PairStore<OutT>::st(po + 2 * plane, v[2]);
        } else {
            PairStore<OutT>::st(po, make_float2(v[0].x, v[1].x));
            PairStore<OutT>::st(po + 2, make_float2(v[2].x, v[0].y));
            PairStore<OutT>::st(po + 4, make_float2(v[1].y, v[2].y));
        }
    } else {
        const size_t cs = LAYOUT == RB200_NCHW ? plane : 1;
        const size_t xs = LAYOUT == RB200_NCHW ? 1 : 3;
        po[0] = OutConv<OutT>::cvt(v[0].x);
        po[cs] = OutConv<OutT>::cvt(v[1].x);
        po[2 * cs] = OutConv<OutT>::cvt(v[2].x);
        if (second) {
            po[xs] = OutConv<OutT>::cvt(v[0].y);
            po[xs + cs] = OutConv<OutT>::cvt(v[1].y);
            po[xs + 2 * cs] = OutConv<OutT>::cvt(v[2].y);
        }
    }
}

template <typename OutT, int LAYOUT, bool NORMALIZE, bool PAIRED>
__device__ __forceinline__ void staged_rows(const uint8_t* stage, const StagedRow* rows, int j_begin, int j_end,
                                            const ColumnTaps (&ct)[2], float2 wx2, float2 owx2, bool second,
                                            const float (&mulv)[3], const float (&addv)[3], const uint32_t magic,
                                            OutT* po, size_t row_step, size_t plane) {
    for (int j = j_begin; j < j_end; j++, po += row_step) {
        const float4 wts = *reinterpret_cast<const float4*>(&rows[j]);
        const int2 offs = *reinterpret_cast<const int2*>(&rows[j].off0);
        blend_store<OutT, LAYOUT, NORMALIZE, PAIRED>(stage, offs.x, offs.y, make_float2(wts.x, wts.y), make_float2(wts.z, wts.w),
                                                     ct, wx2, owx2, second, mulv, addv, magic, po, plane);
    }
}

// Per-thread set-up of the two columns a thread owns.
__device__ __forceinline__ void column_setup(int xi0, bool second, int crop_x, int crop_w, int mirror, float ratio_w,
                                             float off_w, int roi_x, int x_lo, int x_hi, int x_first,
                                             ColumnTaps (&ct)[2], float2& wx2, float2& owx2) {
    float wxs[2], owxs[2];
#pragma unroll
    for (int p = 0; p < 2; p++) {
        int xi = (p == 1 && !second) ? xi0 : xi0 + p;
        int rx = crop_x + (mirror ? (crop_w - 1 - xi) : xi);
        float sx = src_location(rx, ratio_w, off_w, roi_x);
        float fx = floorf(sx);
        wxs[p] = sub_rn(sx, fx);
        owxs[p] = sub_rn(1.0f, wxs[p]);
        int x0, x1;
        clamp_taps(fx, x_lo, x_hi, x0, x1);
        ct[p].o_left = (x0 - x_first) * 3;
        ct[p].same = (x1 == x0);
        ct[p].sel_r = ct[p].same ? 0x7650u : 0x7653u;
        ct[p].sel_g = ct[p].same ? 0x7651u : 0x7650u;
        ct[p].sel_b = ct[p].same ? 0x7652u : 0x7651u;
    }
    wx2 = make_float2(wxs[0], wxs[1]);
    owx2 = make_float2(owxs[0], owxs[1]);
}

// ------------------------------------------------------------------------------------------
// Stream kernel: a CTA owns a strip of `strip_rows` output rows of one tile column of one sample.
// Column set-up happens once per thread for the whole strip. The source rows the strip's taps touch arrive, each
// exactly once, through a ring of 2 NS row slots filled by one producer lane with 1-D bulk copies (cp.async.bulk, the
// TMA unit) that complete on the slot's "full" mbarrier; consumers release a row by arriving on the slot's "empty"
// mbarrier after the last output row that reads it. Every wait is bounded: on a time-out the kernel sets the
// launch's status word, drains the copies it has in flight (bounded again) and returns.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` SM clock cycles (and after 2^24 polls at the latest). The polling loop is kept
// out of line: the callers' fast path is one try_wait.
__device__ __forceinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, long long limit) {
    const long long t0 = clock64();
    for (int i = 0; i < (1 << 24); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) break;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_poll(bar, parity, limit);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int kMaxStripRows = 32;

// ---- pair ring: each stage holds the two tap rows of one output row ------------------------------------------------
// The variant for sources in device memory. A row that two output rows share (down-scale ratios below 2, up-scales) is
// fetched for each of them; in device memory the second fetch is an L2 hit and this ring's simpler bookkeeping (one
// barrier wait and one release per output row) makes it the faster of the two there. Sources in mapped host memory
// use the row ring below, which fetches every row once.
struct PairRow {           // per strip row, built once per CTA (32 bytes + 16 bytes)
    float2 wy2, owy2;
    int off0, off1;          // byte offset of the first staged pixel of the two tap rows (stage included)
    uint32_t b0, b1;         // bytes of the two bulk copies
};
struct PairSrc {
    const uint8_t *g0, *g1;  // 16-byte aligned global sources of the two copies
};

template <typename OutT, int LAYOUT, bool NORMALIZE>
__global__ void __launch_bounds__(288, 4) resample_stream_pairs_kernel(const uint8_t* __restrict__ arena,
                                                              const rb200_resample_sample* __restrict__ samples,
                                                              const ResampleLaunch L) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    if (!L.overlap) pdl_wait();
    // Layout: full[NS] | empty[NS] (128 bytes reserved) | PairRow[32] | PairSrc[32] | stages
    const int NS = L.ns, ns_mask = L.ns - 1, ns_lg = L.ns_log2;
    PairRow* rowtab = reinterpret_cast<PairRow*>(smem + 128);
    PairSrc* srctab = reinterpret_cast<PairSrc*>(smem + 128 + sizeof(PairRow) * kMaxStripRows);
    uint8_t* stage = smem + 128 + (sizeof(PairRow) + sizeof(PairSrc)) * kMaxStripRows;
    const uint32_t bar_base = smem_u32(smem);
    const uint32_t stage_base = smem_u32(stage);

    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int strip = blockIdx.x / L.tiles_x;
    const int tid = threadIdx.x;
    const int TW = 2 * L.twh;
    const int producer_tid = (int)blockDim.x - 32;      // lane 0 of the last warp

    const rb200_resample_sample* sp = samples + n;
    const int crop_w = sp->crop_w, crop_h = sp->crop_h;
    const int cw = min(crop_w, L.out_w);
    const int ch = min(crop_h, L.out_h);
    const int tile_x0 = tx * TW;
    const int y_begin = strip * L.strip_rows;
    const int xi0 = tile_x0 + 2 * tid;
    OutT* out = reinterpret_cast<OutT*>(L.out);

    const int rows_valid = min(L.strip_rows, ch - y_begin);
    const int cols_valid = min(TW, cw - tile_x0);

    // bounds-checking build: a sample whose source rectangle leaves the arena is reported and none of it is read
    const bool src_ok = rect_in_bounds(L.bounds, arena + sp->src_offset, sp->src_stride, sp->roi_x, sp->roi_y, sp->roi_w, sp->roi_h,
                                       L.status);
    if (rows_valid > 0 && cols_valid > 0 && src_ok) {
        const uint8_t* img = arena + sp->src_offset;
        const uint32_t stride = sp->src_stride;
        const int roi_x = sp->roi_x, roi_w = sp->roi_w;
        const int crop_x = sp->crop_x, mirror = sp->mirror;
        const int x_lo = roi_x, x_hi = max(roi_x + roi_w - 2, roi_x);
        const float ratio_w = div_rn((float)roi_w, (float)sp->dst_w);
        const float off_w = mul_rn(sub_rn(ratio_w, 1.0f), 0.5f);
        int x_first, x_last;
        {
            int ca = tile_x0, cb = tile_x0 + cols_valid - 1;
            int ra = crop_x + (mirror ? (crop_w - 1 - ca) : ca);
            int rb = crop_x + (mirror ? (crop_w - 1 - cb) : cb);
            int r_lo = min(ra, rb), r_hi = max(ra, rb);
            int t0, t1;
            clamp_taps(floorf(src_location(r_lo, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
            x_first = t0;
            clamp_taps(floorf(src_location(r_hi, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
            x_last = t1;
        }

        // Row table of the strip (one thread per row) and barrier initialisation.
        if (tid < rows_valid) {
            const int roi_y = sp->roi_y, roi_h = sp->roi_h;
            const float ratio_h = div_rn((float)roi_h, (float)sp->dst_h);
            const float off_h = mul_rn(sub_rn(ratio_h, 1.0f), 0.5f);
            const int y_lo = roi_y, y_hi = max(roi_y + roi_h - 2, roi_y);
            const int nbytes = (x_last - x_first + 1) * 3;
            const int s = tid & ns_mask;
            float sy = src_location(sp->crop_y + y_begin + tid, ratio_h, off_h, roi_y);
            float fy = floorf(sy);
            int y0, y1;
            clamp_taps(fy, y_lo, y_hi, y0, y1);
            const uint8_t* g0 = img + (size_t)y0 * stride + (size_t)x_first * 3;
            const uint8_t* g1 = img + (size_t)y1 * stride + (size_t)x_first * 3;
            const uint32_t m0 = (uint32_t)((uintptr_t)g0 & 15), m1 = (uint32_t)((uintptr_t)g1 & 15);
            float wy = sub_rn(sy, fy), owy = sub_rn(1.0f, wy);
            PairRow r;
            r.wy2 = make_float2(wy, wy);
            r.owy2 = make_float2(owy, owy);
            r.off0 = (2 * s) * L.pitch + (int)m0;
            r.off1 = (2 * s + 1) * L.pitch + (int)m1;
            r.b0 = ((m0 + nbytes + 15) >> 4) << 4;
            r.b1 = ((m1 + nbytes + 15) >> 4) << 4;
            rowtab[tid] = r;
            srctab[tid].g0 = g0 - m0;
            srctab[tid].g1 = g1 - m1;
        }
        if (tid == producer_tid) {
            for (int s = 0; s < NS; s++) {
                mbar_init(bar_base + 8 * s, 1);                   // full: one arrive (+ tx bytes)
                mbar_init(bar_base + 8 * (NS + s), L.twh);        // empty: every compute thread
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();

        if (tid >= producer_tid) {
            // ---- producer warp: lane 0 keeps the ring full ----
            if (tid == producer_tid) {
                for (int j = 0; j < rows_valid; j++) {
                    const int s = j & ns_mask;
                    if (j == L.skip_row) break;        // self-test: this row's copies (and all later ones) never start
                    if (j >= NS && !mbar_wait_bounded(bar_base + 8 * (NS + s), ((j >> ns_lg) - 1) & 1, L.wait_cycles)) {
                        raise_status(L.status);
                        break;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    const uint2 bytes = *reinterpret_cast<const uint2*>(&rowtab[j].b0);
                    const PairSrc src = srctab[j];
                    const uint32_t bar = bar_base + 8 * s;
                    if (!span_in_bounds(L.bounds, src.g0, bytes.x, L.status) || !span_in_bounds(L.bounds, src.g1, bytes.y, L.status))
                        break;                         // (bounds-checking build) the copy is not made; the consumers give up
                    mbar_expect_tx(bar, bytes.x + bytes.y);
                    bulk_g2s(stage_base + (2 * s) * L.pitch, src.g0, bytes.x, bar);
                    bulk_g2s(stage_base + (2 * s + 1) * L.pitch, src.g1, bytes.y, bar);
                }
            }
        } else if (tid < L.twh) {
            // ---- compute threads ----
            const bool active = 2 * tid < cols_valid;
            const bool second = (2 * tid + 1) < cols_valid;
            ColumnTaps ct[2];
            float2 wx2, owx2;
            column_setup(active ? xi0 : tile_x0, second, crop_x, crop_w, mirror, ratio_w, off_w, roi_x, x_lo, x_hi, x_first, ct, wx2, owx2);
            const size_t plane = (size_t)L.out_w * L.out_h;
            OutT* po = out + out_index<OutT, LAYOUT>(L.out_w, L.out_h, n, 0, y_begin, active ? xi0 : tile_x0);
            const size_t row_step = LAYOUT == RB200_NCHW ? (size_t)L.out_w : (size_t)L.out_w * 3;
            const bool paired = second && L.pair_ok;
            // The row loop is written out per kind of warp, so that the common one (every lane owns two columns, none at
            // the image border) tests nothing but the barrier and carries no border selects. The choice is made per warp
            // (votes over the lanes that are here), never per lane: all lanes of a warp stay in one loop.
            int j = 0;
            bool ok = true;
            auto rows_loop = [&](auto kind) {
                constexpr int KIND = decltype(kind)::value;      // 0 idle, 1 mixed, 2 full + border lanes, 3 full
                for (; j < rows_valid; j++, po += row_step) {
                    const int s = j & ns_mask;
                    if (!mbar_wait_bounded(bar_base + 8 * s, (j >> ns_lg) & 1, L.wait_cycles)) {
                        ok = false;
                        break;
                    }
                    if (KIND != 0 && (KIND != 1 || active)) {
                        const float4 wts = *reinterpret_cast<const float4*>(&rowtab[j]);
                        const int2 offs = *reinterpret_cast<const int2*>(&rowtab[j].off0);
                        if (KIND != 1 || paired)
                            blend_store<OutT, LAYOUT, NORMALIZE, true, KIND != 3>(
                                stage, offs.x, offs.y, make_float2(wts.x, wts.y), make_float2(wts.z, wts.w), ct, wx2, owx2,
                                second, L.mul, L.add, L.magic, po, plane);
                        else
                            blend_store<OutT, LAYOUT, NORMALIZE, false, true>(
                                stage, offs.x, offs.y, make_float2(wts.x, wts.y), make_float2(wts.z, wts.w), ct, wx2, owx2,
                                second, L.mul, L.add, L.magic, po, plane);
                    }
                    mbar_arrive(bar_base + 8 * (NS + s));
                }
            };
            const unsigned lanes = __activemask();
            const bool none_active = !__any_sync(lanes, active);
            const bool all_full = __all_sync(lanes, active && paired);
            const bool border = __any_sync(lanes, active && (ct[0].same || ct[1].same));
            if (none_active) rows_loop(std::integral_constant<int, 0>());
            else if (!all_full) rows_loop(std::integral_constant<int, 1>());
            else if (border) rows_loop(std::integral_constant<int, 2>());
            else rows_loop(std::integral_constant<int, 3>());
            if (!ok) {
                raise_status(L.status);
                // Before the CTA's shared memory is given away, wait (bounded) for the copies that may
                // still be in flight: the producer is never more than NS rows ahead.
                if (tid == 0)
                    for (int jj = j; jj < min(j + NS, rows_valid); jj++)
                        mbar_wait_bounded(bar_base + 8 * (jj & ns_mask), (jj >> ns_lg) & 1, L.wait_cycles);
            }
        }
    }

    if (L.fill_padding && tid < L.twh) {
        const int j_end = min(L.strip_rows, L.out_h - y_begin);
        for (int jj = 0; jj < j_end; jj++) {
            int y = y_begin + jj;
#pragma unroll
            for (int p = 0; p < 2; p++) {
                int xi = xi0 + p;
                if (xi < L.out_w && (y >= ch || xi >= cw)) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
            }
        }
    }
    if (L.overlap) pdl_wait();      // completion of this launch implies completion of the kernel before it
}


// ---- row ring: every distinct source row of the strip is fetched once --------------------------------------------
struct StreamRow {           // per output row of the strip, built once per CTA (32 bytes)
    float2 wy2, owy2;
    int off0, off1;          // byte offset of the first staged pixel of the two tap rows (slot and alignment included)
    uint32_t ctl;            // what the consumer needs per row, ready to use: bits 0-7 / 8-15 byte offset of the "full"
                             // barrier of the top / bottom tap row's slot (the "empty" one lies 64 bytes further),
                             // bit 16 / 17 the phase parity to wait for, bit 18 the bottom row is another row than the
                             // top one, bits 20-21 how many rows (0..2, top first) no later output row needs
    int u0;                  // index of the top tap row in the strip's list of distinct source rows
};
struct StreamSrc {           // per distinct source row of the strip (16 bytes)
    const uint8_t* g;        // 16-byte aligned global source of the copy
    uint32_t bytes;          // bytes of the copy (a multiple of 16)
    uint32_t pad;
};
constexpr size_t kStreamTableBytes = sizeof(StreamRow) * kMaxStripRows + sizeof(StreamSrc) * 2 * kMaxStripRows;

// The strip's two tables, by one warp (lane = output row of the strip): per output row the vertical weights, where its
// two tap rows lie in the ring and which rows it releases; per distinct source row the copy the producer issues.
// The tap rows never decrease from one output row to the next and the bottom tap is the top tap or the row below it,
// so a lane only has to look at its predecessor's bottom row to know which of its rows are new. Kept out of line so
// that its registers do not add to those of the pixel loop.
__device__ __noinline__ void build_strip_tables(const rb200_resample_sample* __restrict__ sp, const uint8_t* __restrict__ img,
                                                int x_first, int nbytes, int y_begin, int rows_valid, int smask, int slog,
                                                int pitch, StreamRow* rowtab, StreamSrc* srctab, int* distinct_out) {
    const int tid = threadIdx.x;
    const bool have = tid < rows_valid;
    const uint32_t stride = sp->src_stride;
    const int roi_y = sp->roi_y, roi_h = sp->roi_h;
    const float ratio_h = div_rn((float)roi_h, (float)sp->dst_h);
    const float off_h = mul_rn(sub_rn(ratio_h, 1.0f), 0.5f);
    const int y_lo = roi_y, y_hi = max(roi_y + roi_h - 2, roi_y);
    float sy = src_location(sp->crop_y + y_begin + min(tid, rows_valid - 1), ratio_h, off_h, roi_y);
    float fy = floorf(sy);
    int y0, y1;
    clamp_taps(fy, y_lo, y_hi, y0, y1);
    const int py1 = __shfl_up_sync(0xffffffffu, y1, 1);
    const bool first = tid == 0;
    const int new0 = (have && (first || y0 > py1)) ? 1 : 0;
    const int new1 = (have && y1 > y0 && (first || y1 > py1)) ? 1 : 0;
    const int cnt = new0 + new1;
    int inc = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (tid >= d) inc += t;
    }
    const int before = inc - cnt;          // distinct rows listed before this output row's new ones
    const int u0 = new0 ? before : before - 1 - (py1 - y0);
    const int u1 = (y1 == y0) ? u0 : (new1 ? before + new0 : before - 1 - (py1 - y1));
    const int total = __shfl_sync(0xffffffffu, inc, rows_valid - 1);
    const int u0_next = __shfl_down_sync(0xffffffffu, u0, 1);
    if (have) {
        const uint8_t* g0 = img + (size_t)y0 * stride + (size_t)x_first * 3;
        const uint8_t* g1 = img + (size_t)y1 * stride + (size_t)x_first * 3;
        const uint32_t m0 = (uint32_t)((uintptr_t)g0 & 15), m1 = (uint32_t)((uintptr_t)g1 & 15);
        float wy = sub_rn(sy, fy), owy = sub_rn(1.0f, wy);
        StreamRow r;
        r.wy2 = make_float2(wy, wy);
        r.owy2 = make_float2(owy, owy);
        r.off0 = (u0 & smask) * pitch + (int)m0;
        r.off1 = (u1 & smask) * pitch + (int)m1;
        const int rel = (tid == rows_valid - 1) ? total - u0 : u0_next - u0;
        r.ctl = (uint32_t)((u0 & smask) * 8) | ((uint32_t)((u1 & smask) * 8) << 8) | ((uint32_t)((u0 >> slog) & 1) << 16) |
                ((uint32_t)((u1 >> slog) & 1) << 17) | ((u1 != u0) ? (1u << 18) : 0u) | ((uint32_t)rel << 20);
        r.u0 = u0;
        rowtab[tid] = r;
        if (new0) {
            srctab[before].g = g0 - m0;
            srctab[before].bytes = ((m0 + nbytes + 15) >> 4) << 4;
        }
        if (new1) {
            srctab[before + new0].g = g1 - m1;
            srctab[before + new0].bytes = ((m1 + nbytes + 15) >> 4) << 4;
        }
    }
    if (tid == 0) *distinct_out = total;
}

// The ring holds source rows, each fetched once: the rows the strip's taps touch, in ascending order, form a list of
// distinct rows (skipped rows of a strong down-scale are not in it; a row that two or more output rows share - every
// down-scale ratio below 2, every up-scale - is in it once). Row u of the list lives in slot u mod (2 NS). An output
// row waits for the one or two slots of its tap rows and, when done, releases the rows that no later output row needs.
template <typename OutT, int LAYOUT, bool NORMALIZE>
__global__ void __launch_bounds__(288, 4) resample_stream_kernel(const uint8_t* __restrict__ arena,
                                                              const rb200_resample_sample* __restrict__ samples,
                                                              const ResampleLaunch L) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_distinct;
    pdl_launch_dependents();
    if (!L.overlap) pdl_wait();
    // Layout: full[slots] (64 bytes) | empty[slots] (64 bytes) | StreamRow[32] | StreamSrc[64] | row slots
    const int slots = 2 * L.ns, smask = slots - 1, slog = L.ns_log2 + 1;
    StreamRow* rowtab = reinterpret_cast<StreamRow*>(smem + 128);
    StreamSrc* srctab = reinterpret_cast<StreamSrc*>(smem + 128 + sizeof(StreamRow) * kMaxStripRows);
    uint8_t* stage = smem + 128 + kStreamTableBytes;
    const uint32_t full_base = smem_u32(smem), empty_base = smem_u32(smem + 64);
    const uint32_t stage_base = smem_u32(stage);

    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int strip = blockIdx.x / L.tiles_x;
    const int tid = threadIdx.x;
    const int TW = 2 * L.twh;
    const int producer_tid = (int)blockDim.x - 32;      // lane 0 of the last warp

    const rb200_resample_sample* sp = samples + n;
    const int crop_w = sp->crop_w, crop_h = sp->crop_h;
    const int cw = min(crop_w, L.out_w);
    const int ch = min(crop_h, L.out_h);
    const int tile_x0 = tx * TW;
    const int y_begin = strip * L.strip_rows;
    const int xi0 = tile_x0 + 2 * tid;
    OutT* out = reinterpret_cast<OutT*>(L.out);

    const int rows_valid = min(L.strip_rows, ch - y_begin);
    const int cols_valid = min(TW, cw - tile_x0);

    // bounds-checking build: a sample whose source rectangle leaves the arena is reported and none of it is read
    const bool src_ok = rect_in_bounds(L.bounds, arena + sp->src_offset, sp->src_stride, sp->roi_x, sp->roi_y, sp->roi_w, sp->roi_h,
                                       L.status);
    if (rows_valid > 0 && cols_valid > 0 && src_ok) {
        const uint8_t* img = arena + sp->src_offset;
        const int roi_x = sp->roi_x, roi_w = sp->roi_w;
        const int crop_x = sp->crop_x, mirror = sp->mirror;
        const int x_lo = roi_x, x_hi = max(roi_x + roi_w - 2, roi_x);
        const float ratio_w = div_rn((float)roi_w, (float)sp->dst_w);
        const float off_w = mul_rn(sub_rn(ratio_w, 1.0f), 0.5f);
        int x_first, x_last;
        {
            int ca = tile_x0, cb = tile_x0 + cols_valid - 1;
            int ra = crop_x + (mirror ? (crop_w - 1 - ca) : ca);
            int rb = crop_x + (mirror ? (crop_w - 1 - cb) : cb);
            int r_lo = min(ra, rb), r_hi = max(ra, rb);
            int t0, t1;
            clamp_taps(floorf(src_location(r_lo, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
            x_first = t0;
            clamp_taps(floorf(src_location(r_hi, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
            x_last = t1;
        }

        // Row tables of the strip, by the first warp (one lane per output row), and barrier initialisation.
        if (tid < 32)
            build_strip_tables(sp, img, x_first, (x_last - x_first + 1) * 3, y_begin, rows_valid, smask, slog, L.pitch, rowtab,
                               srctab, &s_distinct);
        if (tid == producer_tid) {
            for (int s = 0; s < slots; s++) {
                mbar_init(full_base + 8 * s, 1);                  // full: one arrive (+ tx bytes)
                mbar_init(empty_base + 8 * s, (L.twh + 31) >> 5); // empty: one arrive per compute warp
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncthreads();

        if (tid >= producer_tid) {
            // ---- producer warp: lane 0 keeps the ring full ----
            if (tid == producer_tid) {
                const int distinct = s_distinct;
                for (int u = 0; u < distinct; u++) {
                    const int s = u & smask;
                    if (u == L.skip_row) break;        // self-test: this row's copy (and all later ones) never starts
                    if (u >= slots && !mbar_wait_bounded(empty_base + 8 * s, ((u >> slog) - 1) & 1, L.wait_cycles)) {
                        raise_status(L.status);
                        break;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    const StreamSrc src = srctab[u];
                    const uint32_t bar = full_base + 8 * s;
                    if (!span_in_bounds(L.bounds, src.g, src.bytes, L.status))
                        break;                         // (bounds-checking build) the copy is not made; the consumers give up
                    mbar_expect_tx(bar, src.bytes);
                    bulk_g2s(stage_base + s * L.pitch, src.g, src.bytes, bar);
                }
            }
        } else if (tid < L.twh) {
            // ---- compute threads ----
            const bool active = 2 * tid < cols_valid;
            const bool second = (2 * tid + 1) < cols_valid;
            ColumnTaps ct[2];
            float2 wx2, owx2;
            column_setup(active ? xi0 : tile_x0, second, crop_x, crop_w, mirror, ratio_w, off_w, roi_x, x_lo, x_hi, x_first, ct, wx2, owx2);
            const size_t plane = (size_t)L.out_w * L.out_h;
            OutT* po = out + out_index<OutT, LAYOUT>(L.out_w, L.out_h, n, 0, y_begin, active ? xi0 : tile_x0);
            const size_t row_step = LAYOUT == RB200_NCHW ? (size_t)L.out_w : (size_t)L.out_w * 3;
            const bool paired = second && L.pair_ok;
            // the compute lanes of this warp (the last warp may be half full: twh is a multiple of 16)
            const int lanes = min(32, L.twh - (tid & ~31));
            const unsigned wmask = lanes == 32 ? 0xffffffffu : ((1u << lanes) - 1u);
            const bool releaser = (tid & 31) == 0;
            int j = 0, u_fail = 0;
            bool ok = true;
            for (; j < rows_valid; j++, po += row_step) {
                const int4 info = *reinterpret_cast<const int4*>(&rowtab[j].off0);     // off0, off1, ctl, u0
                const uint32_t ctl = (uint32_t)info.z;
                ok = mbar_wait_bounded(full_base + (ctl & 0xffu), (ctl >> 16) & 1u, L.wait_cycles);
                if (ok && (ctl & (1u << 18))) ok = mbar_wait_bounded(full_base + ((ctl >> 8) & 0xffu), (ctl >> 17) & 1u, L.wait_cycles);
                // a warp gives up as a whole: its lanes meet again at the release below
                ok = __all_sync(wmask, ok) != 0;
                if (!ok) {
                    u_fail = info.w;
                    break;
                }
                if (active) {
                    const float4 wts = *reinterpret_cast<const float4*>(&rowtab[j]);
                    if (paired)
                        blend_store<OutT, LAYOUT, NORMALIZE, true>(stage, info.x, info.y, make_float2(wts.x, wts.y), make_float2(wts.z, wts.w),
                                                                   ct, wx2, owx2, second, L.mul, L.add, L.magic, po, plane);
                    else
                        blend_store<OutT, LAYOUT, NORMALIZE, false>(stage, info.x, info.y, make_float2(wts.x, wts.y), make_float2(wts.z, wts.w),
                                                                    ct, wx2, owx2, second, L.mul, L.add, L.magic, po, plane);
                }
                // release the rows no later output row reads, once per warp after all its lanes have read them (the
                // "empty" barriers lie 64 bytes behind the "full" ones)
                if (ctl & (3u << 20)) {
                    __syncwarp(wmask);
                    if (releaser) {
                        mbar_arrive(full_base + 64 + (ctl & 0xffu));
                        if (ctl & (2u << 20)) mbar_arrive(full_base + 64 + ((ctl >> 8) & 0xffu));
                    }
                }
            }
            if (!ok) {
                raise_status(L.status);
                // Before the CTA's shared memory is given away, wait (bounded) for the copies that may
                // still be in flight: the producer is never more than the ring's slots ahead.
                if (tid == 0) {
                    const int distinct = s_distinct;
                    for (int u = u_fail; u < min(u_fail + slots, distinct); u++)
                        mbar_wait_bounded(full_base + 8 * (u & smask), (u >> slog) & 1, L.wait_cycles);
                }
            }
        }
    }

    if (L.fill_padding && tid < L.twh) {
        const int j_end = min(L.strip_rows, L.out_h - y_begin);
        for (int jj = 0; jj < j_end; jj++) {
            int y = y_begin + jj;
#pragma unroll
            for (int p = 0; p < 2; p++) {
                int xi = xi0 + p;
                if (xi < L.out_w && (y >= ch || xi >= cw)) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
            }
        }
    }
    if (L.overlap) pdl_wait();      // completion of this launch implies completion of the kernel before it
}

template <typename OutT, int LAYOUT, bool NORMALIZE>
__global__ void __launch_bounds__(256) resample_staged_kernel(const uint8_t* __restrict__ arena,
                                                              const rb200_resample_sample* __restrict__ samples,
                                                              const ResampleLaunch L) {
    extern __shared__ __align__(128) uint8_t smem[];
    // Layout: TileHeader | StagedRow[th] | int srow[2*th+2] | (16-byte aligned) staged rows
    TileHeader* hdr = reinterpret_cast<TileHeader*>(smem);
    StagedRow* rows = reinterpret_cast<StagedRow*>(smem + sizeof(TileHeader));
    int* srow = reinterpret_cast<int*>(smem + sizeof(TileHeader) + sizeof(StagedRow) * L.th);
    uint8_t* stage = smem + ((sizeof(TileHeader) + sizeof(StagedRow) * L.th + sizeof(int) * (2 * L.th + 2) + 15) & ~(size_t)15);

    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int tid = threadIdx.x;
    const int nthreads = blockDim.x;
    const int TW = 2 * L.twh;

    const rb200_resample_sample* sp = samples + n;
    const int crop_w = sp->crop_w, crop_h = sp->crop_h;
    const int cw = min(crop_w, L.out_w);
    const int ch = min(crop_h, L.out_h);
    const int tile_x0 = tx * TW;
    const int tile_y0 = ty * L.th;
    int grp = 0, col = tid;
    if (L.groups > 1) { grp = tid / L.twh; col = tid - grp * L.twh; }
    const int xi0 = tile_x0 + 2 * col;
    const int rpg = L.th / L.groups;                    // rows per row group
    const int j_begin = grp * rpg;
    OutT* out = reinterpret_cast<OutT*>(L.out);

    const int rows_valid = min(L.th, ch - tile_y0);     // rows of this tile inside the crop
    const int cols_valid = min(TW, cw - tile_x0);       // columns of this tile inside the crop

    // bounds-checking build: a sample whose source rectangle leaves the arena is reported and none of it is read
    const bool src_ok = rect_in_bounds(L.bounds, arena + sp->src_offset, sp->src_stride, sp->roi_x, sp->roi_y, sp->roi_w, sp->roi_h,
                                       L.status);
    if (rows_valid > 0 && cols_valid > 0 && src_ok) {
        const uint8_t* img = arena + sp->src_offset;
        const uint32_t stride = sp->src_stride;
        const int roi_x = sp->roi_x, roi_w = sp->roi_w;
        const int crop_x = sp->crop_x, mirror = sp->mirror;
        const int x_lo = roi_x;
        const int x_hi = max(roi_x + roi_w - 2, roi_x);

        // Warp 0 builds the tile header (lane 0) and the row table (lanes < rows_valid).
        if (tid < 32) {
            const int roi_y = sp->roi_y, roi_h = sp->roi_h, crop_y = sp->crop_y;
            const float ratio_h = div_rn((float)roi_h, (float)sp->dst_h);
            const float off_h = mul_rn(sub_rn(ratio_h, 1.0f), 0.5f);
            const float ratio_w = div_rn((float)roi_w, (float)sp->dst_w);
            const float off_w = mul_rn(sub_rn(ratio_w, 1.0f), 0.5f);
            const int y_lo = roi_y, y_hi = max(roi_y + roi_h - 2, roi_y);
            // Source column range of the tile.
            int x_first, x_last;
            {
                int ca = tile_x0, cb = tile_x0 + cols_valid - 1;
                int ra = crop_x + (mirror ? (crop_w - 1 - ca) : ca);
                int rb = crop_x + (mirror ? (crop_w - 1 - cb) : cb);
                int r_lo = min(ra, rb), r_hi = max(ra, rb);
                int t0, t1;
                clamp_taps(floorf(src_location(r_lo, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
                x_first = t0;
                clamp_taps(floorf(src_location(r_hi, ratio_w, off_w, roi_x)), x_lo, x_hi, t0, t1);
                x_last = t1;
            }
            // Rows are staged as one contiguous range when consecutive output rows share source
            // rows (ratio <= 2), else as one pair per output row.
            const bool dense = !(ratio_h > 2.0f);
            int y_first = 0, nslots = 2 * rows_valid;
            if (dense) {
                int t0, t1;
                clamp_taps(floorf(src_location(crop_y + tile_y0, ratio_h, off_h, roi_y)), y_lo, y_hi, t0, t1);
                y_first = t0;
                clamp_taps(floorf(src_location(crop_y + tile_y0 + rows_valid - 1, ratio_h, off_h, roi_y)), y_lo, y_hi, t0, t1);
                nslots = t1 - y_first + 1;
            }
            if (tid == 0) {
                hdr->ratio_w = ratio_w;
                hdr->off_w = off_w;
                hdr->x_first = x_first;
                hdr->nbytes = (x_last - x_first + 1) * 3;
                hdr->nslots = nslots;
            }
            if (tid < rows_valid) {
                float sy = src_location(crop_y + tile_y0 + tid, ratio_h, off_h, roi_y);
                float fy = floorf(sy);
                int y0, y1;
                clamp_taps(fy, y_lo, y_hi, y0, y1);
                StagedRow ri;
                float wy = sub_rn(sy, fy), owy = sub_rn(1.0f, wy);
                ri.wy2 = make_float2(wy, wy);
                ri.owy2 = make_float2(owy, owy);
                int s0 = dense ? (y0 - y_first) : 2 * tid;
                int s1 = dense ? (y1 - y_first) : 2 * tid + 1;
                uint32_t m0 = (uint32_t)((uintptr_t)(img + (size_t)y0 * stride + (size_t)x_first * 3) & 15);
                uint32_t m1 = (uint32_t)((uintptr_t)(img + (size_t)y1 * stride + (size_t)x_first * 3) & 15);
                ri.off0 = s0 * L.pitch + (int)m0;
                ri.off1 = s1 * L.pitch + (int)m1;
                ri.pad[0] = ri.pad[1] = 0;
                if (!dense) { srow[2 * tid] = y0; srow[2 * tid + 1] = y1; }
                rows[tid] = ri;
            }
            if (dense) {
                for (int r = tid; r < nslots; r += 32) srow[r] = y_first + r;
            }
        }
        __syncthreads();
        const float ratio_w = hdr->ratio_w, off_w = hdr->off_w;
        const int x_first = hdr->x_first;

        // Stage: one warp per source row, 16 bytes per lane and step.
        {
            const int nbytes = hdr->nbytes, nslots = hdr->nslots;
            const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
            // a trailing partial warp (block sizes are multiples of 16) takes no rows
            for (int r = warp < nwarps ? warp : nslots; r < nslots; r += nwarps) {
                const uint8_t* g = img + (size_t)srow[r] * stride + (size_t)x_first * 3;
                const uint32_t m = (uint32_t)((uintptr_t)g & 15);
                const int need = (int)(m + nbytes + 15) >> 4;
                const uint8_t* ga = g - m;
                uint8_t* sd = stage + (size_t)r * L.pitch;
                if (!span_in_bounds(L.bounds, ga, (size_t)need * 16, L.status)) continue;   // (bounds-checking build)
                for (int ck = lane; ck < need; ck += 32) cp_async16(sd + ck * 16, ga + ck * 16);
            }
            cp_async_commit_wait_all();
            __syncthreads();
        }

        if (2 * col < cols_valid && j_begin < rows_valid) {
            const bool second = (2 * col + 1) < cols_valid;
            ColumnTaps ct[2];
            float wxs[2], owxs[2];
#pragma unroll
            for (int p = 0; p < 2; p++) {
                int xi = (p == 1 && !second) ? xi0 : xi0 + p;
                int rx = crop_x + (mirror ? (crop_w - 1 - xi) : xi);
                float sx = src_location(rx, ratio_w, off_w, roi_x);
                float fx = floorf(sx);
                wxs[p] = sub_rn(sx, fx);
                owxs[p] = sub_rn(1.0f, wxs[p]);
                int x0, x1;
                clamp_taps(fx, x_lo, x_hi, x0, x1);
                ct[p].o_left = (x0 - x_first) * 3;
                ct[p].same = (x1 == x0);
                ct[p].sel_r = ct[p].same ? 0x7650u : 0x7653u;
                ct[p].sel_g = ct[p].same ? 0x7651u : 0x7650u;
                ct[p].sel_b = ct[p].same ? 0x7652u : 0x7651u;
            }
            const float2 wx2 = make_float2(wxs[0], wxs[1]);
            const float2 owx2 = make_float2(owxs[0], owxs[1]);
            const size_t plane = (size_t)L.out_w * L.out_h;
            OutT* po = out + out_index<OutT, LAYOUT>(L.out_w, L.out_h, n, 0, tile_y0 + j_begin, xi0);
            const size_t row_step = LAYOUT == RB200_NCHW ? (size_t)L.out_w : (size_t)L.out_w * 3;
            const int j_end = min(j_begin + rpg, rows_valid);
            if (second && L.pair_ok)
                staged_rows<OutT, LAYOUT, NORMALIZE, true>(stage, rows, j_begin, j_end, ct, wx2, owx2, second, L.mul, L.add, L.magic, po, row_step, plane);
            else
                staged_rows<OutT, LAYOUT, NORMALIZE, false>(stage, rows, j_begin, j_end, ct, wx2, owx2, second, L.mul, L.add, L.magic, po, row_step, plane);
        }
    }

    if (L.fill_padding) {
        // Zero the part of the tile that lies outside the sample's valid extent.
        const int j_end = min(j_begin + rpg, L.out_h - tile_y0);
        for (int j = j_begin; j < j_end; j++) {
            int y = tile_y0 + j;
#pragma unroll
            for (int p = 0; p < 2; p++) {
                int xi = xi0 + p;
                if (xi < L.out_w && (y >= ch || xi >= cw)) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
            }
        }
    }
}

// Direct variant: one thread per output column, taps read from global memory.
template <typename OutT, int LAYOUT>
__global__ void __launch_bounds__(256) resample_direct_kernel(const uint8_t* __restrict__ arena,
                                                              const rb200_resample_sample* __restrict__ samples,
                                                              const ResampleLaunch L) {
    __shared__ RowInfo rowinfo[8];
    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int tid = threadIdx.x;
    const int TW = blockDim.x;

    const rb200_resample_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);

    const int cw = min(s.crop_w, L.out_w);
    const int ch = min(s.crop_h, L.out_h);
    const int tile_x0 = tx * TW;
    const int tile_y0 = ty * L.th;
    const int xi = tile_x0 + tid;
    const int rows_valid = min(L.th, ch - tile_y0);
    const int cols_valid = min(TW, cw - tile_x0);

    const bool src_ok = rect_in_bounds(L.bounds, img, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status);
    if (rows_valid > 0 && cols_valid > 0 && src_ok) {
        const float ratio_w = div_rn((float)s.roi_w, (float)s.dst_w);
        const float ratio_h = div_rn((float)s.roi_h, (float)s.dst_h);
        const float off_w = mul_rn(sub_rn(ratio_w, 1.0f), 0.5f);
        const float off_h = mul_rn(sub_rn(ratio_h, 1.0f), 0.5f);
        const int x_lo = s.roi_x, y_lo = s.roi_y;
        const int x_hi = max(s.roi_x + s.roi_w - 2, s.roi_x);
        const int y_hi = max(s.roi_y + s.roi_h - 2, s.roi_y);
        if (tid < rows_valid) {
            float sy = src_location(s.crop_y + tile_y0 + tid, ratio_h, off_h, s.roi_y);
            float fy = floorf(sy);
            RowInfo ri;
            clamp_taps(fy, y_lo, y_hi, ri.off0, ri.off1);
            ri.wy = sub_rn(sy, fy);
            ri.owy = sub_rn(1.0f, ri.wy);
            rowinfo[tid] = ri;
        }
        __syncthreads();
        if (tid < cols_valid) {
            int rx = s.crop_x + (s.mirror ? (s.crop_w - 1 - xi) : xi);
            float sx = src_location(rx, ratio_w, off_w, s.roi_x);
            float fx = floorf(sx);
            float wx = sub_rn(sx, fx);
            float owx = sub_rn(1.0f, wx);
            int x0, x1;
            clamp_taps(fx, x_lo, x_hi, x0, x1);
            const int oL = x0 * 3, oR = x1 * 3;
            for (int j = 0; j < rows_valid; j++) {
                const RowInfo ri = rowinfo[j];
                const uint8_t* r0 = img + (size_t)ri.off0 * s.src_stride;
                const uint8_t* r1 = img + (size_t)ri.off1 * s.src_stride;
                const float w00 = mul_rn(ri.owy, owx), w01 = mul_rn(ri.owy, wx), w10 = mul_rn(ri.wy, owx);
                float v[3];
#pragma unroll
                for (int c = 0; c < 3; c++) {
                    float ftl = (float)__ldg(r0 + oL + c), ftr = (float)__ldg(r0 + oR + c);
                    float fbl = (float)__ldg(r1 + oL + c), fbr = (float)__ldg(r1 + oR + c);
                    float acc = mul_rn(mul_rn(fbr, ri.wy), wx);
                    acc = fmaf(fbl, w10, acc);
                    acc = fmaf(ftr, w01, acc);
                    acc = fmaf(ftl, w00, acc);
                    v[c] = sat_round_u8f(acc);
                    if (L.normalize) v[c] = fmaf(v[c], L.mul[c], L.add[c]);
                }
                store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, tile_y0 + j, xi, v[0], v[1], v[2]);
            }
        }
    }
    if (L.fill_padding && xi < L.out_w) {
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int j = 0; j < rows_in_tile; j++) {
            int y = tile_y0 + j;
            if (y >= ch || xi >= cw) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
        }
    }
}

// ---- triangular ("generic") interpolation -------------------------------------------------------
// One thread per output column, th rows per CTA, taps gathered through L1/L2. Arithmetic of
// resize_generic_pln1_hip_tensor (rocAL/rocAL_hip/rocal_hip_kernels.cpp:487-589) on each channel:
// per axis radius = max(ratio, 1), scale = 1/radius, ceil(2*radius) taps starting at
// ceil(dst*ratio + (ratio-1)/2 - radius + roi), triangle weights max(0, 1 - |(w - radius + j)*scale|),
// rows outer / columns inner accumulation with one fmaf per tap and channel, normalisation by
// 1 / (row_sum * col_sum), clamp to [0,255] and truncation.
struct TriAxis {
    float radius, scale, offset;
    int ksize;
};
__device__ __forceinline__ TriAxis tri_axis_make(float ratio) {
    TriAxis a;
    if (ratio > 1.0f) { a.radius = ratio; a.scale = div_rn(1.0f, ratio); } else { a.radius = 1.0f; a.scale = 1.0f; }
    a.offset = sub_rn(mul_rn(sub_rn(ratio, 1.0f), 0.5f), a.radius);
    a.ksize = (int)ceilf(mul_rn(a.radius, 2.0f));
    return a;
}
__device__ __forceinline__ void tri_loc(const TriAxis& a, float ratio, int dst, int roi_lo, int limit, int& first, float& weight) {
    const float raw = add_rn(fmaf((float)dst, ratio, a.offset), (float)roi_lo);
    const int r = (int)ceilf(raw);
    weight = sub_rn((float)r, raw);
    first = min(r, limit);
}
__device__ __forceinline__ float tri_coeff(const TriAxis& a, float weight, int j) {
    const float c = sub_rn(1.0f, fabsf(mul_rn(add_rn(sub_rn(weight, a.radius), (float)j), a.scale)));
    return c < 0.f ? 0.f : c;
}

// Accumulates the KX taps of one source row. The column coefficients and (for threads at the image border) the
// clamped byte offsets do not depend on the row, so they live in registers.
//
// INTERIOR (every tap inside the ROI): the taps are 3*KX contiguous bytes. They are fetched as the aligned 32-bit
// words that contain them (each word holds at least one needed byte, so no load leaves the mapped page of the last
// pixel), brought to byte 0 by funnel shifts, and turned into floats by PRMT into the mantissa of 2^23 plus one
// packed subtraction per two bytes - no byte loads and no integer-to-float conversion unit, which were the two
// busiest units of the byte-wise version. Border threads keep byte loads with the same conversion.
template <int KX, bool INTERIOR>
__device__ __forceinline__ void tri_row(const uint8_t* __restrict__ r, const float (&cc)[KX], const int (&coff)[KX], float rc,
                                        float& acc0, float& acc1, float& acc2) {
    if (INTERIOR) {
        constexpr int NB = 3 * KX;               // bytes of the taps
        constexpr int NV = (NB + 3) / 4;         // aligned words after the shift
        constexpr int NW = (NB + 3 + 3) / 4;     // words to fetch when the first byte sits at offset 3
        const unsigned sb = (unsigned)(reinterpret_cast<uintptr_t>(r) & 3u);
        const uint32_t* ab = reinterpret_cast<const uint32_t*>(r - sb);
        uint32_t w[NW + 1];
#pragma unroll
        for (int i = 0; i < NW; i++) w[i] = (4 * i < (int)sb + NB) ? __ldg(ab + i) : 0u;
        w[NW] = 0u;
        uint32_t v[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) v[i] = __funnelshift_r(w[i], w[i + 1], sb * 8);
        float x[NB + 1];
#pragma unroll
        for (int t = 0; t < NB; t += 2) {
            float2 p;
            p.x = __uint_as_float(__byte_perm(v[t / 4], 0x4B000000u, 0x7650u + (t % 4)));
            p.y = t + 1 < NB ? __uint_as_float(__byte_perm(v[(t + 1) / 4], 0x4B000000u, 0x7650u + ((t + 1) % 4))) : 8388608.0f;
            p = add2(p, make_float2(-8388608.0f, -8388608.0f));
            x[t] = p.x;
            x[t + 1] = p.y;
        }
#pragma unroll
        for (int k = 0; k < KX; k++) {
            const float coeff = mul_rn(cc[k], rc);
            acc0 = fmaf(x[3 * k], coeff, acc0);
            acc1 = fmaf(x[3 * k + 1], coeff, acc1);
            acc2 = fmaf(x[3 * k + 2], coeff, acc2);
        }
    } else {
#pragma unroll
        for (int k = 0; k < KX; k++) {
            const uint8_t* px = r + coff[k];
            const float coeff = mul_rn(cc[k], rc);
            acc0 = fmaf(sub_rn(__uint_as_float(0x4B000000u | __ldg(px)), 8388608.0f), coeff, acc0);
            acc1 = fmaf(sub_rn(__uint_as_float(0x4B000000u | __ldg(px + 1)), 8388608.0f), coeff, acc1);
            acc2 = fmaf(sub_rn(__uint_as_float(0x4B000000u | __ldg(px + 2)), 8388608.0f), coeff, acc2);
        }
    }
}

// All output rows of one thread for a column filter of exactly KX taps (KX = 0: any tap count, nothing hoisted).
template <typename OutT, int LAYOUT, int KX>
__device__ __forceinline__ void tri_column(const uint8_t* __restrict__ img, const rb200_resample_sample& s, const ResampleLaunch& L,
                                           OutT* out, int n, int xi, int tile_y0, int rows_valid, const TriAxis& ax,
                                           const TriAxis& ay, float ratio_w, float ratio_h) {
    const int x_lo = s.roi_x, y_lo = s.roi_y;
    const int x_hi = s.roi_x + s.roi_w - 1, y_hi = s.roi_y + s.roi_h - 1;
    const int rx = s.crop_x + (s.mirror ? (s.crop_w - 1 - xi) : xi);
    int fx;
    float wx;
    tri_loc(ax, ratio_w, rx, x_lo, x_hi, fx, wx);
    constexpr int KA = KX > 0 ? KX : 1;
    float cc[KA];
    int coff[KA];
    float col_sum_fixed = 0.f;
    bool interior = false;
    if (KX > 0) {
#pragma unroll
        for (int k = 0; k < KA; k++) {
            cc[k] = tri_coeff(ax, wx, k);
            col_sum_fixed = add_rn(col_sum_fixed, cc[k]);
            coff[k] = min(max(fx + k, x_lo), x_hi) * 3;
        }
        interior = fx >= x_lo && fx + KX - 1 <= x_hi;
    }
    for (int j0 = 0; j0 < rows_valid; j0++) {
        int fy;
        float wy;
        tri_loc(ay, ratio_h, s.crop_y + tile_y0 + j0, y_lo, y_hi, fy, wy);
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, row_sum = 0.f, col_sum = col_sum_fixed;
        for (int j = 0; j < ay.ksize; j++) {
            const int row = min(max(fy + j, y_lo), y_hi);
            const uint8_t* r = img + (size_t)row * s.src_stride;
            const float rc = tri_coeff(ay, wy, j);
            row_sum = add_rn(row_sum, rc);
            if (KX > 0) {
                if (interior)
                    tri_row<KA, true>(r + fx * 3, cc, coff, rc, acc0, acc1, acc2);
                else
                    tri_row<KA, false>(r, cc, coff, rc, acc0, acc1, acc2);
            } else {
                col_sum = 0.f;
                for (int k = 0; k < ax.ksize; k++) {
                    const int col = min(max(fx + k, x_lo), x_hi);
                    const float c1 = tri_coeff(ax, wx, k);
                    col_sum = add_rn(col_sum, c1);
                    const float coeff = mul_rn(c1, rc);
                    const uint8_t* px = r + col * 3;
                    acc0 = fmaf((float)__ldg(px), coeff, acc0);
                    acc1 = fmaf((float)__ldg(px + 1), coeff, acc1);
                    acc2 = fmaf((float)__ldg(px + 2), coeff, acc2);
                }
            }
        }
        if (row_sum == 0.f) row_sum = 1.f;
        if (col_sum == 0.f) col_sum = 1.f;
        const float inv = div_rn(1.0f, mul_rn(row_sum, col_sum));
        float v[3] = {mul_rn(acc0, inv), mul_rn(acc1, inv), mul_rn(acc2, inv)};
#pragma unroll
        for (int c = 0; c < 3; c++) {
            v[c] = truncf(fmaxf(fminf(v[c], 255.f), 0.f));     // fmaxf sends NaN to 0
            if (L.normalize) v[c] = fmaf(v[c], L.mul[c], L.add[c]);
        }
        store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, tile_y0 + j0, xi, v[0], v[1], v[2]);
    }
}

// The other filters of the resize family on the same skeleton (weight functions and base radii of this library's
// own choosing, see rb200_kernels.h): radius = B * max(ratio, 1), scale = 1 / max(ratio, 1), the weight function
// evaluated at (weight - radius + j) * scale. Same operation order as the CPU restatement; lanczos and gaussian go
// through sinf / expf, which differ from the host's by rounding.
__device__ __forceinline__ TriAxis filter_axis_make(float ratio, int filter) {
    if (filter == RB200_INTERP_TRIANGULAR) return tri_axis_make(ratio);
    const float base = filter == RB200_INTERP_BICUBIC ? 2.0f : (filter == RB200_INTERP_LANCZOS ? 3.0f : (filter == RB200_INTERP_NEAREST ? 0.5f : 1.0f));
    TriAxis a;
    a.radius = mul_rn(base, ratio > 1.0f ? ratio : 1.0f);
    a.scale = ratio > 1.0f ? div_rn(1.0f, ratio) : 1.0f;
    a.offset = sub_rn(mul_rn(sub_rn(ratio, 1.0f), 0.5f), a.radius);
    a.ksize = max(1, (int)ceilf(mul_rn(a.radius, 2.0f)));
    return a;
}
__device__ __forceinline__ float filter_weight(int filter, float x) {
    const float ax = fabsf(x);
    if (filter == RB200_INTERP_BICUBIC) {
        if (ax >= 2.0f) return 0.f;
        if (ax > 1.0f) return add_rn(fmaf(-4.0f, ax, mul_rn(mul_rn(ax, ax), fmaf(-0.5f, ax, 2.5f))), 2.0f);
        return fmaf(mul_rn(ax, ax), fmaf(1.5f, ax, -2.5f), 1.0f);
    }
    if (filter == RB200_INTERP_LANCZOS) {
        if (ax >= 3.0f) return 0.f;
        if (ax < 1e-5f) return 1.0f;
        const float px = mul_rn(ax, 3.14159265358979323846f);
        return div_rn(mul_rn(3.0f, mul_rn(sinf(px), sinf(mul_rn(px, 1.0f / 3.0f)))), mul_rn(px, px));
    }
    if (filter == RB200_INTERP_GAUSSIAN) return expf(mul_rn(-4.0f, mul_rn(x, x)));
    if (filter == RB200_INTERP_NEAREST) return 1.0f;
    const float c = sub_rn(1.0f, ax);
    return c < 0.f ? 0.f : c;
}
__device__ __forceinline__ float filter_coeff(const TriAxis& a, int filter, float weight, int j) {
    return filter_weight(filter, mul_rn(add_rn(sub_rn(weight, a.radius), (float)j), a.scale));
}

// All output rows of one thread for a filter chosen at run time (nothing hoisted).
template <typename OutT, int LAYOUT>
__device__ __forceinline__ void filter_column(const uint8_t* __restrict__ img, const rb200_resample_sample& s, const ResampleLaunch& L,
                                              OutT* out, int n, int xi, int tile_y0, int rows_valid, const TriAxis& ax,
                                              const TriAxis& ay, float ratio_w, float ratio_h) {
    const int x_lo = s.roi_x, y_lo = s.roi_y;
    const int x_hi = s.roi_x + s.roi_w - 1, y_hi = s.roi_y + s.roi_h - 1;
    const int rx = s.crop_x + (s.mirror ? (s.crop_w - 1 - xi) : xi);
    int fx;
    float wx;
    tri_loc(ax, ratio_w, rx, x_lo, x_hi, fx, wx);
    for (int j0 = 0; j0 < rows_valid; j0++) {
        int fy;
        float wy;
        tri_loc(ay, ratio_h, s.crop_y + tile_y0 + j0, y_lo, y_hi, fy, wy);
        float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, row_sum = 0.f, col_sum = 0.f;
        for (int j = 0; j < ay.ksize; j++) {
            const int row = min(max(fy + j, y_lo), y_hi);
            const uint8_t* r = img + (size_t)row * s.src_stride;
            const float rc = filter_coeff(ay, L.filter, wy, j);
            row_sum = add_rn(row_sum, rc);
            col_sum = 0.f;
            for (int k = 0; k < ax.ksize; k++) {
                const int col = min(max(fx + k, x_lo), x_hi);
                const float c1 = filter_coeff(ax, L.filter, wx, k);
                col_sum = add_rn(col_sum, c1);
                const float coeff = mul_rn(c1, rc);
                const uint8_t* px = r + col * 3;
                acc0 = fmaf((float)__ldg(px), coeff, acc0);
                acc1 = fmaf((float)__ldg(px + 1), coeff, acc1);
                acc2 = fmaf((float)__ldg(px + 2), coeff, acc2);
            }
        }
        if (row_sum == 0.f) row_sum = 1.f;
        if (col_sum == 0.f) col_sum = 1.f;
        const float inv = div_rn(1.0f, mul_rn(row_sum, col_sum));
        float v[3] = {mul_rn(acc0, inv), mul_rn(acc1, inv), mul_rn(acc2, inv)};
#pragma unroll
        for (int c = 0; c < 3; c++) {
            v[c] = truncf(fmaxf(fminf(v[c], 255.f), 0.f));     // fmaxf sends NaN to 0
            if (L.normalize) v[c] = fmaf(v[c], L.mul[c], L.add[c]);
        }
        store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, tile_y0 + j0, xi, v[0], v[1], v[2]);
    }
}

template <typename OutT, int LAYOUT>
__global__ void __launch_bounds__(256) resample_triangular_kernel(const uint8_t* __restrict__ arena,
                                                                  const rb200_resample_sample* __restrict__ samples,
                                                                  const ResampleLaunch L) {
    const int n = blockIdx.y;
    const int tx = blockIdx.x % L.tiles_x;
    const int ty = blockIdx.x / L.tiles_x;
    const int xi = tx * blockDim.x + threadIdx.x;
    const int tile_y0 = ty * L.th;

    const rb200_resample_sample s = samples[n];
    const uint8_t* img = arena + s.src_offset;
    OutT* out = reinterpret_cast<OutT*>(L.out);
    const int cw = min(s.crop_w, L.out_w);
    const int ch = min(s.crop_h, L.out_h);
    const int rows_valid = min(L.th, ch - tile_y0);

    const bool src_ok = rect_in_bounds(L.bounds, img, s.src_stride, s.roi_x, s.roi_y, s.roi_w, s.roi_h, L.status);
    if (rows_valid > 0 && xi < cw && src_ok) {
        const float ratio_w = div_rn((float)s.roi_w, (float)s.dst_w);
        const float ratio_h = div_rn((float)s.roi_h, (float)s.dst_h);
        const TriAxis ax = filter_axis_make(ratio_w, L.filter), ay = filter_axis_make(ratio_h, L.filter);
        if (L.filter != RB200_INTERP_TRIANGULAR) {
            filter_column<OutT, LAYOUT>(img, s, L, out, n, xi, tile_y0, rows_valid, ax, ay, ratio_w, ratio_h);
        } else
        // the tap count is the same for the whole sample, so this switch does not diverge
        switch (ax.ksize) {
#define RB200_TRI_CASE(K) \
    case K: tri_column<OutT, LAYOUT, K>(img, s, L, out, n, xi, tile_y0, rows_valid, ax, ay, ratio_w, ratio_h); break;
            RB200_TRI_CASE(2) RB200_TRI_CASE(3) RB200_TRI_CASE(4) RB200_TRI_CASE(5) RB200_TRI_CASE(6) RB200_TRI_CASE(7)
            RB200_TRI_CASE(8)
#undef RB200_TRI_CASE
            default: tri_column<OutT, LAYOUT, 0>(img, s, L, out, n, xi, tile_y0, rows_valid, ax, ay, ratio_w, ratio_h); break;
        }
    }
    if (L.fill_padding && xi < L.out_w) {
        const int rows_in_tile = min(L.th, L.out_h - tile_y0);
        for (int j = 0; j < rows_in_tile; j++) {
            int y = tile_y0 + j;
            if (y >= ch || xi >= cw) store3<OutT, LAYOUT>(out, L.out_w, L.out_h, n, y, xi, 0.f, 0.f, 0.f);
        }
    }
}

enum { MODE_DIRECT = 0, MODE_STAGED = 1, MODE_STREAM = 2, MODE_TRIANGULAR = 3 };

// CTAs of `kernel` the whole device holds at once for this block size and shared-memory request (asked of the
// runtime once per combination).
static long resident_ctas(const void* kernel, int threads, size_t smem) {
    struct Entry { const void* k; int threads; size_t smem; int dev; long ctas; };
    static std::mutex m;
    static std::vector<Entry> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(m);
    for (const Entry& e : cache)
        if (e.k == kernel && e.threads == threads && e.smem == smem && e.dev == dev) return e.ctas;
    int per_sm = 0, sms = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm <= 0) {
        cudaGetLastError();
        per_sm = 4;
    }
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        cudaGetLastError();
        sms = 148;
    }
    cache.push_back({kernel, threads, smem, dev, (long)per_sm * sms});
    return cache.back().ctas;
}

// Output rows per CTA of the row-streaming kernel. Strips are balanced (ceil(ext_h / k) rows for a whole number k of
// strips, so no CTA gets a short leftover). A grid of at least four waves at 32 rows keeps 32 (least set-up per row).
// Smaller grids are latency-bound - a CTA's life is its set-up plus one copy round trip per ring refill - and run
// fastest with about 14 rows per CTA (measured on 64 .. 256 images of 224 rows: 14 beats 8, 16 and 32 by 3 .. 40 %);
// grids that would not even fill half the device at 14 rows go down to 8.
// A source in host memory is a different case: the launch is bound by the link, not by latency, and every strip border
// makes two CTAs pull the rows their taps share, so the tallest strips win as soon as the grid keeps the link busy
// (measured on 64 images: 32 rows 396 us, 14 rows 404 us, 8 rows 412 us).
static int choose_strip_rows(long resident, long columns_of_ctas, int ext_h, bool host_source) {
    auto ctas_at = [&](int rows) { return columns_of_ctas * ((ext_h + rows - 1) / rows); };
    int target = 14;
    if (ctas_at(32) >= 4 * resident || (host_source && ctas_at(32) * 3 >= resident)) target = 32;
    else if (ctas_at(14) * 2 < resident) target = 8;
    int k = (ext_h + target / 2) / target;
    if (k < 1) k = 1;
    int rows = (ext_h + k - 1) / k;
    if (rows > kMaxStripRows) rows = kMaxStripRows;
    if (rows < 4) rows = ext_h < 4 ? ext_h : 4;
    return rows < 1 ? 1 : rows;
}

template <typename OutT, int LAYOUT>
static int launch_typed(const uint8_t* arena, const rb200_resample_sample* samples, int n, ResampleLaunch L,
                        int mode, size_t smem, cudaStream_t stream) {
    L.pair_ok = (L.out_w % 2 == 0) && (((uintptr_t)L.out) % (2 * sizeof(OutT)) == 0);
    if (mode == MODE_STREAM) {
        auto k = L.row_ring ? (L.normalize ? resample_stream_kernel<OutT, LAYOUT, true> : resample_stream_kernel<OutT, LAYOUT, false>)
                            : (L.normalize ? resample_stream_pairs_kernel<OutT, LAYOUT, true>
                                           : resample_stream_pairs_kernel<OutT, LAYOUT, false>);
        if (smem > 48 * 1024) {
            int rc = check_cuda(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                "cudaFuncSetAttribute(resample_stream)");
            if (rc) return rc;
        }
        // compute threads rounded up to whole warps + one producer warp
        const int threads = ((L.twh + 31) & ~31) + 32;
        if (L.strip_rows == 0) L.strip_rows = choose_strip_rows(resident_ctas((const void*)k, threads, smem), n * L.tiles_x, L.ext_h, L.row_ring != 0);
        int strips = (L.ext_h + L.strip_rows - 1) / L.strip_rows;
        dim3 grid((unsigned)(L.tiles_x * strips), (unsigned)n);
        cudaError_t le = launch_overlapped(k, grid, dim3((unsigned)threads), smem, stream, arena, samples, L);
        if (le != cudaSuccess) return check_cuda(le, "launch of resample_stream_kernel");
    } else if (mode == MODE_STAGED) {
        int tiles_y = (L.ext_h + L.th - 1) / L.th;
        dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
        auto k = L.normalize ? resample_staged_kernel<OutT, LAYOUT, true> : resample_staged_kernel<OutT, LAYOUT, false>;
        if (smem > 48 * 1024) {
            int rc = check_cuda(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                                "cudaFuncSetAttribute(resample)");
            if (rc) return rc;
        }
        k<<<grid, L.twh * L.groups, smem, stream>>>(arena, samples, L);
    } else {
        int tx = (L.ext_w + 255) / 256;
        int tw = ((L.ext_w + tx - 1) / tx + 31) & ~31;
        L.tiles_x = (L.ext_w + tw - 1) / tw;
        L.th = 8;
        int tiles_y = (L.ext_h + L.th - 1) / L.th;
        dim3 grid((unsigned)(L.tiles_x * tiles_y), (unsigned)n);
        if (mode == MODE_TRIANGULAR)
            resample_triangular_kernel<OutT, LAYOUT><<<grid, tw, 0, stream>>>(arena, samples, L);
        else
            resample_direct_kernel<OutT, LAYOUT><<<grid, tw, 0, stream>>>(arena, samples, L);
    }
    RB200_CHECK_LAUNCH("resample_kernel");
    return RB200_OK;
}

}  // namespace rb200

using namespace rb200;

static int resample_launch(const uint8_t* arena, const rb200_resample_sample* samples,
                           const rb200_resample_sample* h_samples, int n, const rb200_resample_params* p,
                           void* stream_v, unsigned long long wait_cycles, int skip_row) {
    if (n == 0) return RB200_OK;
    if (!arena || !samples || !p || !p->out || n < 0 || p->out_w <= 0 || p->out_h <= 0) {
        set_error("rb200k_resample: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (n > 65535) {
        set_error("rb200k_resample: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (p->out_dtype < 0 || p->out_dtype > 2 || (p->out_layout != RB200_NCHW && p->out_layout != RB200_NHWC)) {
        set_error("rb200k_resample: bad out_dtype %d / out_layout %d", p->out_dtype, p->out_layout);
        return RB200_E_INVALID;
    }
    if (p->interpolation < RB200_INTERP_BILINEAR || p->interpolation > RB200_INTERP_NEAREST) {
        set_error("rb200k_resample: bad interpolation %d", p->interpolation);
        return RB200_E_INVALID;
    }
    if (p->strip_rows != 0 && (p->strip_rows < 4 || p->strip_rows > kMaxStripRows)) {
        set_error("rb200k_resample: strip_rows %d is outside 4..%d", p->strip_rows, kMaxStripRows);
        return RB200_E_INVALID;
    }
    if (p->path < RB200_RESAMPLE_PATH_AUTO || p->path > RB200_RESAMPLE_PATH_PAIRS) {
        set_error("rb200k_resample: bad path %d", p->path);
        return RB200_E_INVALID;
    }
    cudaStream_t stream = (cudaStream_t)stream_v;

    ResampleLaunch L;
    L.filter = p->interpolation;
    L.out = p->out;
    L.out_w = p->out_w;
    L.out_h = p->out_h;
    L.normalize = p->normalize;
    L.fill_padding = p->fill_padding;
    L.pair_ok = 0;
    L.magic = 0x4B000000u;
    for (int c = 0; c < 3; c++) { L.mul[c] = p->mul[c]; L.add[c] = p->add[c]; }
    L.status = p->status ? p->status : default_status_word();
    if (!L.status) {
        set_error("rb200k_resample: the device's status word cannot be addressed");
        return RB200_E_CUDA;
    }
    L.wait_cycles = (long long)(wait_cycles ? wait_cycles : kDefaultWaitCycles);
    L.skip_row = skip_row;
    L.overlap = p->overlap ? 1 : 0;
    // Which ring the row-streaming kernel runs: every source row once for a source in host memory (each re-read would
    // cross the link again), tap-row pairs for device memory (re-reads are L2 hits and the bookkeeping is lighter).
    L.row_ring = p->path == RB200_RESAMPLE_PATH_ROWS;
    if (p->path == RB200_RESAMPLE_PATH_AUTO) {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, arena) == cudaSuccess) L.row_ring = attr.type == cudaMemoryTypeHost;
        else cudaGetLastError();
    }
    L.bounds = arena_bounds(arena, p->arena_bytes);
    if (p->out_bytes && (uint64_t)n * p->out_w * p->out_h * 3 * out_elem_size(p->out_dtype) > p->out_bytes) {
        set_error("rb200k_resample: %d samples of %d x %d x 3 elements do not fit the %llu-byte output", n, p->out_w, p->out_h,
                  (unsigned long long)p->out_bytes);
        return RB200_E_INVALID;
    }

    // Extent the grid has to cover.
    int ext_w = p->out_w, ext_h = p->out_h;
    if (h_samples) {
        for (int i = 0; i < n; i++) {
            if (h_samples[i].dst_w <= 0 || h_samples[i].dst_h <= 0 || h_samples[i].roi_w <= 0 || h_samples[i].roi_h <= 0) {
                set_error("rb200k_resample: sample %d has an empty roi or target size", i);
                return RB200_E_INVALID;
            }
        }
    }
    if (h_samples && !p->fill_padding) {
        ext_w = 1; ext_h = 1;
        for (int i = 0; i < n; i++) {
            int w = h_samples[i].crop_w < p->out_w ? h_samples[i].crop_w : p->out_w;
            int h = h_samples[i].crop_h < p->out_h ? h_samples[i].crop_h : p->out_h;
            if (w > ext_w) ext_w = w;
            if (h > ext_h) ext_h = h;
        }
    }
    L.ext_w = ext_w;
    L.ext_h = ext_h;

    // Staged geometry: tiles of <= 512 columns, two columns per thread, 1..8 row groups per CTA.
    bool staged = h_samples != nullptr;
    int th = 8, pitch = 0;
    L.tiles_x = (ext_w + 511) / 512;
    int tile_px = (ext_w + L.tiles_x - 1) / L.tiles_x;
    int twh = (((tile_px + 1) / 2) + 15) & ~15;
    // Every thread keeps its column set-up for all rows of its group, so one group per CTA is
    // preferred; narrow tiles take more groups to reach at least 64 threads.
    int groups = 1;
    while (groups < 8 && twh * groups < 64) groups *= 2;
    L.tiles_x = (ext_w + 2 * twh - 1) / (2 * twh);
    int mode = staged ? MODE_STAGED : MODE_DIRECT;
    size_t smem = 0;
    L.strip_rows = 32;
    L.ns = 4;
    L.ns_log2 = 2;
    if (staged) {
        int max_span = 1;
        for (int i = 0; i < n; i++) {
            double ratio = (double)h_samples[i].roi_w / (double)h_samples[i].dst_w;
            long span = (long)(2.0 * twh * ratio) + 4;
            if (span > h_samples[i].roi_w) span = h_samples[i].roi_w;
            if (span > max_span) max_span = (int)span;
        }
        pitch = (15 + max_span * 3 + 12 + 15) & ~15;
        // Wide tiles stream their rows through the bulk-copy ring; narrow ones use the tile kernel.
        bool want_stream = twh >= 64 && p->path != RB200_RESAMPLE_PATH_TILE;
        if (want_stream) {
            int ns = 4;
            if ((size_t)2 * ns * pitch > 96 * 1024) ns = 2;
            if ((size_t)2 * ns * pitch <= 160 * 1024) {
                mode = MODE_STREAM;
                L.ns = ns;
                L.ns_log2 = ns == 4 ? 2 : 1;
                L.strip_rows = p->strip_rows;      // 0: chosen in launch_typed, where the kernel's occupancy is known
                smem = 128 + kStreamTableBytes + (size_t)2 * ns * pitch;
            }
        }
        if (mode == MODE_STAGED) {
            const size_t budget = 40 * 1024, hard = 160 * 1024;
            while (th > groups && (size_t)(2 * th + 2) * pitch > budget) th >>= 1;
            while (groups > th) groups >>= 1;
            if ((size_t)(2 * th + 2) * pitch > hard) mode = MODE_DIRECT;
            smem = ((sizeof(TileHeader) + sizeof(StagedRow) * th + sizeof(int) * (2 * th + 2) + 15) & ~(size_t)15) +
                   (size_t)(2 * th + 2) * pitch;
        }
    }
    if (p->interpolation != RB200_INTERP_BILINEAR) mode = MODE_TRIANGULAR;   // the generic-filter kernel
    L.th = th;
    L.pitch = pitch;
    L.twh = twh;
    L.groups = groups;

#define RB200_DISPATCH(T, LAY) return launch_typed<T, LAY>(arena, samples, n, L, mode, smem, stream)
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

extern "C" int rb200k_resample(const uint8_t* arena, const rb200_resample_sample* samples,
                               const rb200_resample_sample* h_samples, int n, const rb200_resample_params* p,
                               void* stream_v) {
    return resample_launch(arena, samples, h_samples, n, p, stream_v, kDefaultWaitCycles, -1);
}

extern "C" int rb200k_resample_probe(const uint8_t* arena, const rb200_resample_sample* samples,
                                     const rb200_resample_sample* h_samples, int n, const rb200_resample_params* p,
                                     void* stream_v, uint64_t wait_cycles, int skip_row) {
    return resample_launch(arena, samples, h_samples, n, p, stream_v, wait_cycles, skip_row);
}
