// SSD box encoder: one thread-block cluster of 8 CTAs per sample. Each CTA owns an eighth of the
// anchors and keeps them, their areas and the per-anchor running best in registers; the per-box argmax
// over the anchors is a warp-shuffle reduction, a scan over the CTA's warps and a scan over the eight
// CTAs' results read through distributed shared memory. The winner's "forced match" is an atomicMax
// into the shared memory of the CTA that owns that anchor. Splitting a sample over a cluster (rather
// than one large CTA per sample) gives 8 x batch work items, so the ragged box counts balance over the
// 148 SMs; batches of up to 512 samples are also taken longest sample first.
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
// cluster until the final coalesced write.
#include <cooperative_groups.h>

#include "box_common.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace rb200 {

constexpr int kCluster = 8;     // CTAs per sample (the portable maximum cluster size)
constexpr int kBoxChunk = 64;   // boxes reduced per round of cluster barriers
constexpr int kMaxWarps = 16;   // CTAs have at most 512 threads

struct BoxLaunch {
    const float4* anchors;
    int num_anchors;
    int per_cta;        // anchors owned by one CTA of the cluster
    float criteria;
    float means[4];
    float inv_stds[4];
    int offset;
    float scale, half_scale;
};

// Larger value wins, lower anchor index among equals (the CPU loop's strict '>' over ascending anchors).
__device__ __forceinline__ bool beats(float ov, int oi, float tv, int ti) {
    return ov > tv || (ov == tv && oi < ti);
}

// One box against this thread's K anchors, then the warp's argmax for the box into part_val/part_idx[j].
// Slots past the CTA's share hold an all-zero anchor and are masked to -inf after the IoU, so the loop
// over the slots has no branch.
template <int K, bool FIRST>
__device__ __forceinline__ void box_step(const float4 b, int j, int box, const float4 (&anc)[K], const float (&area_a)[K],
                                         const bool (&valid)[K], float (&best_iou)[K], int (&best_box)[K], int a0,
                                         int nthreads, int lane, int warp, float (*part_val)[kMaxWarps],
                                         int (*part_idx)[kMaxWarps]) {
    float area_b = mul_rn(sub_rn(b.w, b.y), sub_rn(b.z, b.x));
    asm volatile("" : "+f"(area_b));      // computed once per box: the value is opaque from here on, so it is kept, not recomputed per anchor
    float tv = -INFINITY;
    int ti = 0x7fffffff;
#pragma unroll
    for (int k = 0; k < K; k++) {
        float v = iou_ltrb(b, area_b, anc[k], area_a[k]);
        // per anchor: >= over ascending boxes
        if (FIRST || v >= best_iou[k]) { best_iou[k] = v; best_box[k] = box; }
        // per box: strict > over ascending anchors, seeded with anchor 0 (slot 0 of the thread that has a0 == 0)
        v = valid[k] ? v : -INFINITY;
        if ((k == 0 && a0 == 0) || v > tv) { tv = v; ti = a0 + k * nthreads; }
    }
    // Warp argmax with two redux instructions: the value as an order-preserving integer key, then the
    // lowest anchor index among the lanes that hold the maximum. A thread's candidate is NaN only when it
    // is anchor 0's seed, which the CPU loop never replaces: NaN takes the highest key.
    uint32_t key = float_key(tv);
    if (tv != tv) key = 0xffffffffu;
    const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
    ti = (int)__reduce_min_sync(0xffffffffu, key == kmax ? (uint32_t)ti : 0xffffffffu);
    if (key == kmax) {      // every holder of the maximum writes the same pair
        part_val[j][warp] = tv;
        part_idx[j][warp] = ti;
    }
}

// K = anchors per thread: per_cta <= K * blockDim.x.
template <int K>
__global__ void __launch_bounds__((K == 4 ? 320 : 512), (K == 4 ? 4 : 1)) box_encode_kernel(const float4* __restrict__ boxes,
                                                          const int* __restrict__ labels,
                                                          const int* __restrict__ box_offsets,
                                                          float4* __restrict__ out_boxes,
                                                          int* __restrict__ out_labels, const BoxLaunch L) {
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // forced[la] = highest box index whose best anchor is this CTA's local anchor la, or -1
    int* forced = reinterpret_cast<int*>(smem_raw);                      // [K * blockDim.x]
    __shared__ float part_val[kBoxChunk][kMaxWarps];
    __shared__ int part_idx[kBoxChunk][kMaxWarps];
    __shared__ float cta_val[kBoxChunk];     // read by the other CTAs of the cluster
    __shared__ int cta_idx[kBoxChunk];
    __shared__ float4 sbox[kBoxChunk];

    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int A = L.num_anchors;
    const int a_base = rank * L.per_cta;
    const int n = pick_sample(box_offsets, &part_idx[0][0]);
    const int b_begin = box_offsets[n], nb = box_offsets[n + 1] - b_begin;

    float4 anc[K];
    float area_a[K];
    float best_iou[K];
    int best_box[K];
    bool valid[K];
#pragma unroll
    for (int k = 0; k < K; k++) {
        const int la = tid + k * nthreads;
        valid[k] = la < L.per_cta && a_base + la < A;
        anc[k] = valid[k] ? L.anchors[a_base + la] : make_float4(0.f, 0.f, 0.f, 0.f);
        area_a[k] = mul_rn(sub_rn(anc[k].w, anc[k].y), sub_rn(anc[k].z, anc[k].x));
        asm volatile("" : "+f"(area_a[k]));   // likewise: one register per anchor instead of three operations per pair
        best_iou[k] = -1.f;
        best_box[k] = 0;
        forced[la] = -1;
    }
    // every CTA's forced[] is initialised before any CTA of the cluster may write into it
    cluster.sync();

    for (int c0 = 0; c0 < nb; c0 += kBoxChunk) {
        const int cn = min(kBoxChunk, nb - c0);
        if (tid < cn) sbox[tid] = boxes[b_begin + c0 + tid];
        __syncthreads();
        // The first box of a sample takes every anchor's slot whatever its IoU (the CPU loop starts from
        // box 0, NaN included); it is peeled so that the other boxes need no test for it.
        int j = 0;
        if (c0 == 0) {
            box_step<K, true>(sbox[0], 0, 0, anc, area_a, valid, best_iou, best_box, a_base + tid, nthreads, lane, warp,
                              part_val, part_idx);
            j = 1;
        }
        for (; j < cn; j++)
            box_step<K, false>(sbox[j], j, c0 + j, anc, area_a, valid, best_iou, best_box, a_base + tid, nthreads, lane,
                               warp, part_val, part_idx);
        __syncthreads();
        // one thread per box scans the CTA's warps (warp 0 first: it holds anchor 0's seed)
        if (tid < cn) {
            float tv = part_val[tid][0];
            int ti = part_idx[tid][0];
            for (int wv = 1; wv < nwarps; wv++) {
                const float ov = part_val[tid][wv];
                const int oi = part_idx[tid][wv];
                if (beats(ov, oi, tv, ti)) { tv = ov; ti = oi; }
            }
            cta_val[tid] = tv;
            cta_idx[tid] = ti;
        }
        cluster.sync();
        // CTA r finishes boxes r, r+8, ...: scan the eight CTAs in anchor order, then mark the winner in
        // the shared memory of the CTA that owns it.
        if (tid < cn && (tid % kCluster) == rank) {
            float tv = *cluster.map_shared_rank(&cta_val[tid], 0);
            int ti = *cluster.map_shared_rank(&cta_idx[tid], 0);
            for (int r = 1; r < kCluster; r++) {
                const float ov = *cluster.map_shared_rank(&cta_val[tid], r);
                const int oi = *cluster.map_shared_rank(&cta_idx[tid], r);
                if (beats(ov, oi, tv, ti)) { tv = ov; ti = oi; }
            }
            if (ti < A) {
                const int owner = ti / L.per_cta;
                atomicMax(cluster.map_shared_rank(&forced[ti - owner * L.per_cta], owner), c0 + tid);
            }
        }
        // remote reads of cta_val/cta_idx and remote writes of forced[] are complete past this barrier
        cluster.sync();
    }

    float4* ob = out_boxes + (size_t)n * A;
    int* ol = out_labels + (size_t)n * A;
#pragma unroll
    for (int k = 0; k < K; k++) {
        if (!valid[k]) continue;
        const int la = tid + k * nthreads;
        const int a = a_base + la;
        const int f = forced[la];
        float iou = best_iou[k];
        int bb = best_box[k];
        if (f >= 0) { iou = 2.0f; bb = f; }
        float4 o;
        int lab = 0;
        const float4 an = anc[k];
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

template <int K>
static int launch_k(const float4* boxes, const int* labels, const int* box_offsets, int n, float4* out_boxes,
                    int* out_labels, const BoxLaunch& L, int threads, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCluster, (unsigned)n, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = sizeof(int) * K * threads;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, box_encode_kernel<K>, boxes, labels, box_offsets, out_boxes,
                                           out_labels, L),
                        "cudaLaunchKernelEx(box_encode_kernel)");
    if (rc) return rc;
    count_launch();
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
    if (p->num_anchors > kCluster * 16 * 512) {
        set_error("rb200k_box_encode: %d anchors exceed the maximum of %d", p->num_anchors, kCluster * 16 * 512);
        return RB200_E_LIMIT;
    }
    if (n > 65535) {
        set_error("rb200k_box_encode: batch %d exceeds 65535", n);
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
    // Anchors per thread: 4 while a CTA of at most 320 threads covers its share (the SSD-300 table: 8732
    // anchors, 288 threads), then 8 and 16 with CTAs of up to 512 threads.
    L.per_cta = (p->num_anchors + kCluster - 1) / kCluster;
    const int K = L.per_cta <= 4 * 320 ? 4 : (L.per_cta <= 8 * 512 ? 8 : 16);
    int threads = (((L.per_cta + K - 1) / K) + 31) & ~31;
    if (threads < kBoxChunk) threads = kBoxChunk;   // one thread per box of a chunk in the reduction steps
    if (K == 4) return launch_k<4>(b4, labels, box_offsets, n, o4, out_labels, L, threads, stream);
    if (K == 8) return launch_k<8>(b4, labels, box_offsets, n, o4, out_labels, L, threads, stream);
    return launch_k<16>(b4, labels, box_offsets, n, o4, out_labels, L, threads, stream);
}
