// SSD box encoder: one CTA of 1024 threads per sample. The anchor table is staged once per CTA in
// shared memory (8732 anchors = 140 KB of the 227 KB an sm_100 CTA may use), the per-anchor
// running best lives in registers, and the per-box argmax over the anchors is a warp-shuffle
// reduction followed by one warp per box over the 32 per-warp partials.
//
// Semantics (and tie rules) of the CPU encoder, rocAL/source/meta_data/bounding_box_graph.cpp:
//   :61-69    IoU = inter / (area_box + area_anchor - inter), float32, one rounding per op
//   :120-136  for every box the anchor with the highest IoU (lowest index among equals) is
//             forced to match it: its IoU becomes 2.0
//   :138-148  every anchor takes the box with the highest IoU, the highest box index among
//             equals (the comparison is >=, boxes visited in ascending order)
//   :173-216  match if IoU > criteria -> label + (offset-)encoded xcycwh, else label 0 and
//             zeros (offset mode) or the anchor itself as xcycwh.
// The reference's HIP kernel (rocAL/rocAL_hip/box_encoder_hip.cpp:123-176) keeps the running
// best in a global scratch buffer and reduces through shared memory; here nothing leaves the
// SM until the final coalesced write.
#include "common.cuh"

namespace rb200 {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr int kBoxChunk = 32;   // boxes whose per-warp partial argmax is buffered at a time

struct BoxLaunch {
    const float4* anchors;
    int num_anchors;
    float criteria;
    float means[4];
    float inv_stds[4];
    int offset;
    float scale, half_scale;
};

__device__ __forceinline__ float iou_ltrb(const float4 b, float area_b, const float4 a, float area_a) {
    float xa = fmaxf(b.x, a.x), ya = fmaxf(b.y, a.y);
    float xb = fminf(b.z, a.z), yb = fminf(b.w, a.w);
    float inter = mul_rn(fmaxf(0.f, sub_rn(xb, xa)), fmaxf(0.f, sub_rn(yb, ya)));
    return div_rn(inter, sub_rn(add_rn(area_b, area_a), inter));
}

// K = anchors per thread (num_anchors <= K * kThreads); SMEM_ANCHORS = anchor table staged in
// shared memory (otherwise it is re-read through L2 for every box).
template <int K, bool SMEM_ANCHORS>
__global__ void __launch_bounds__(kThreads, 1) box_encode_kernel(const float4* __restrict__ boxes,
                                                                 const int* __restrict__ labels,
                                                                 const int* __restrict__ box_offsets,
                                                                 float4* __restrict__ out_boxes,
                                                                 int* __restrict__ out_labels, const BoxLaunch L) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // forced[a] = highest box index whose best anchor is a, or -1
    float4* sanc = reinterpret_cast<float4*>(smem_raw);
    int* forced = reinterpret_cast<int*>(smem_raw + (SMEM_ANCHORS ? sizeof(float4) * K * kThreads : 0));
    float* part_val = reinterpret_cast<float*>(forced + K * kThreads);   // [kBoxChunk][kWarps]
    int* part_idx = reinterpret_cast<int*>(part_val + kBoxChunk * kWarps);
    float4* sbox = reinterpret_cast<float4*>(part_idx + kBoxChunk * kWarps);   // [kBoxChunk]

    const int n = blockIdx.x;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int A = L.num_anchors;
    const int b_begin = box_offsets[n], nb = box_offsets[n + 1] - b_begin;

    float best_iou[K];
    int best_box[K];
#pragma unroll
    for (int k = 0; k < K; k++) {
        int a = tid + k * kThreads;
        if (SMEM_ANCHORS) sanc[a] = a < A ? L.anchors[a] : make_float4(0.f, 0.f, 0.f, 0.f);
        best_iou[k] = -1.f;
        best_box[k] = 0;
        forced[a] = -1;
    }

    for (int c0 = 0; c0 < nb; c0 += kBoxChunk) {
        const int cn = min(kBoxChunk, nb - c0);
        __syncthreads();   // previous chunk's partials consumed; forced[] initialised
        if (tid < cn) sbox[tid] = boxes[b_begin + c0 + tid];
        __syncthreads();
        for (int j = 0; j < cn; j++) {
            const float4 b = sbox[j];
            const float area_b = mul_rn(sub_rn(b.w, b.y), sub_rn(b.z, b.x));
            float tv = -1.f;
            int ti = 0x7fffffff;
#pragma unroll
            for (int k = 0; k < K; k++) {
                int a = tid + k * kThreads;
                if (a < A) {
                    const float4 an = SMEM_ANCHORS ? sanc[a] : L.anchors[a];
                    const float area_a = mul_rn(sub_rn(an.w, an.y), sub_rn(an.z, an.x));
                    float v = iou_ltrb(b, area_b, an, area_a);
                    // per anchor: >= over ascending boxes. The first box always takes the slot
                    // (the CPU loop starts from box 0 whatever its IoU, NaN included).
                    if ((c0 + j) == 0 || v >= best_iou[k]) { best_iou[k] = v; best_box[k] = c0 + j; }
                    // per box: strict > over ascending anchors, seeded with anchor 0.
                    if (a == 0 || v > tv) { tv = v; ti = a; }
                }
            }
            // warp argmax: larger value wins, lower index among equals.
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, tv, off);
                int oi = __shfl_xor_sync(0xffffffffu, ti, off);
                if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
            }
            if (lane == 0) { part_val[j * kWarps + warp] = tv; part_idx[j * kWarps + warp] = ti; }
        }
        __syncthreads();
        // one warp per box finishes the argmax over the 32 partials
        for (int j = warp; j < cn; j += kWarps) {
            float tv = part_val[j * kWarps + lane];
            int ti = part_idx[j * kWarps + lane];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, tv, off);
                int oi = __shfl_xor_sync(0xffffffffu, ti, off);
                if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
            }
            if (lane == 0 && ti < A) atomicMax(&forced[ti], c0 + j);
        }
    }
    __syncthreads();

    float4* ob = out_boxes + (size_t)n * A;
    int* ol = out_labels + (size_t)n * A;
#pragma unroll
    for (int k = 0; k < K; k++) {
        int a = tid + k * kThreads;
        if (a >= A) continue;
        int f = forced[a];
        float iou = best_iou[k];
        int bb = best_box[k];
        if (f >= 0) { iou = 2.0f; bb = f; }
        float4 o;
        int lab = 0;
        const float4 an = SMEM_ANCHORS ? sanc[a] : L.anchors[a];
        if (iou > L.criteria) {
            const float4 b = boxes[b_begin + bb];
            lab = labels[b_begin + bb];
            if (L.offset) {
                float xc = mul_rn(add_rn(b.x, b.z), L.half_scale);
                float yc = mul_rn(add_rn(b.y, b.w), L.half_scale);
                float w = mul_rn(sub_rn(b.z, b.x), L.scale);
                float h = mul_rn(sub_rn(b.w, b.y), L.scale);
                float axc = mul_rn(add_rn(an.x, an.z), L.half_scale);
                float ayc = mul_rn(add_rn(an.y, an.w), L.half_scale);
                float aw = mul_rn(sub_rn(an.z, an.x), L.scale);
                float ah = mul_rn(sub_rn(an.w, an.y), L.scale);
                o.x = mul_rn(sub_rn(div_rn(sub_rn(xc, axc), aw), L.means[0]), L.inv_stds[0]);
                o.y = mul_rn(sub_rn(div_rn(sub_rn(yc, ayc), ah), L.means[1]), L.inv_stds[1]);
                o.z = mul_rn(sub_rn(logf(div_rn(w, aw)), L.means[2]), L.inv_stds[2]);
                o.w = mul_rn(sub_rn(logf(div_rn(h, ah)), L.means[3]), L.inv_stds[3]);
            } else {
                o.x = mul_rn(0.5f, add_rn(b.x, b.z));
                o.y = mul_rn(0.5f, add_rn(b.y, b.w));
                o.z = sub_rn(b.z, b.x);
                o.w = sub_rn(b.w, b.y);
            }
        } else if (L.offset) {
            o = make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            o.x = mul_rn(0.5f, add_rn(an.x, an.z));
            o.y = mul_rn(0.5f, add_rn(an.y, an.w));
            o.z = add_rn(-an.x, an.z);
            o.w = add_rn(-an.y, an.w);
        }
        ob[a] = o;
        ol[a] = lab;
    }
}

template <int K, bool SMEM_ANCHORS>
static int launch_k(const float4* boxes, const int* labels, const int* box_offsets, int n, float4* out_boxes,
                    int* out_labels, const BoxLaunch& L, cudaStream_t stream) {
    size_t smem = (SMEM_ANCHORS ? sizeof(float4) * K * kThreads : 0) + sizeof(int) * K * kThreads + (sizeof(float) + sizeof(int)) * kBoxChunk * kWarps +
                  sizeof(float4) * kBoxChunk;
    auto k = box_encode_kernel<K, SMEM_ANCHORS>;
    if (smem > 48 * 1024) {
        int rc = check_cuda(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                            "cudaFuncSetAttribute(box_encode)");
        if (rc) return rc;
    }
    k<<<n, kThreads, smem, stream>>>(boxes, labels, box_offsets, out_boxes, out_labels, L);
    RB200_CHECK_LAUNCH("box_encode_kernel");
    return RB200_OK;
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_box_encode(const float* boxes, const int32_t* labels, const int32_t* box_offsets, int n,
                                 int max_boxes_per_sample, const rb200_box_encoder_params* p, float* out_boxes,
                                 int32_t* out_labels, void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!boxes || !labels || !box_offsets || !p || !p->anchors || !out_boxes || !out_labels || n < 0 ||
        p->num_anchors <= 0) {
        set_error("rb200k_box_encode: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (max_boxes_per_sample < 1 || max_boxes_per_sample > 1024) {
        set_error("rb200k_box_encode: max_boxes_per_sample %d outside [1,1024]", max_boxes_per_sample);
        return RB200_E_LIMIT;
    }
    if (p->num_anchors > 32 * kThreads) {
        set_error("rb200k_box_encode: %d anchors exceed the maximum of %d", p->num_anchors, 32 * kThreads);
        return RB200_E_LIMIT;
    }
    if (((uintptr_t)boxes | (uintptr_t)p->anchors | (uintptr_t)out_boxes) & 15) {
        set_error("rb200k_box_encode: boxes, anchors and out_boxes must be 16-byte aligned");
        return RB200_E_INVALID;
    }
    BoxLaunch L;
    L.anchors = reinterpret_cast<const float4*>(p->anchors);
    L.num_anchors = p->num_anchors;
    L.criteria = p->criteria;
    for (int k = 0; k < 4; k++) { L.means[k] = p->means[k]; L.inv_stds[k] = p->inv_stds[k]; }
    L.offset = p->offset;
    L.scale = p->scale;
    L.half_scale = (float)(0.5 * (double)p->scale);
    cudaStream_t stream = (cudaStream_t)stream_v;
    const float4* b4 = reinterpret_cast<const float4*>(boxes);
    float4* o4 = reinterpret_cast<float4*>(out_boxes);
    int K = (p->num_anchors + kThreads - 1) / kThreads;
    if (K <= 4) return launch_k<4, true>(b4, labels, box_offsets, n, o4, out_labels, L, stream);
    if (K <= 9) return launch_k<9, true>(b4, labels, box_offsets, n, o4, out_labels, L, stream);
    if (K <= 16) return launch_k<16, false>(b4, labels, box_offsets, n, o4, out_labels, L, stream);
    return launch_k<32, false>(b4, labels, box_offsets, n, o4, out_labels, L, stream);
}
