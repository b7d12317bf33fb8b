// Box IoU matcher (the RetinaNet-style companion of the SSD box encoder): for every anchor the index of
// the ground-truth box with the highest IoU, or -1 / -2 below the low / high thresholds, with the
// "low-quality matches" rule. Semantics of BoundingBoxGraph::update_box_iou_matcher
// (rocAL/source/meta_data/bounding_box_graph.cpp:222-284):
//   :247-251  per anchor: best box by strict '>' from -1 (lowest box index among equals, NaN never matches)
//   :254-256  per box: highest IoU over all anchors by strict '>' from -1
//   :259-264  an anchor whose IoU with some box lies within 1e-6 of that box's maximum keeps its match
//   :268-277  otherwise best IoU < low_threshold -> -1, < high_threshold -> -2.
//
// One thread-block cluster of 8 CTAs per sample, each CTA owning an eighth of the anchors; the anchors go
// through registers in groups of 4 per thread, so any anchor count fits (RetinaNet: 120 087). With
// low-quality matches the per-box maximum needs every anchor first: sweep 1 reduces it (warp redux on an
// order-preserving key, shared-memory atomicMax per box, then a maximum over the eight CTAs read through
// distributed shared memory), sweep 2 recomputes the IoUs against it. Without them sweep 2 runs alone.
#include <cooperative_groups.h>

#include "box_common.cuh"

namespace cg = cooperative_groups;

namespace rb200 {

constexpr int kMatchCluster = 8;
constexpr int kMatchMaxBoxes = 1024;
constexpr int kMatchK = 4;          // anchors per thread per group

struct MatchLaunch {
    const float4* anchors;
    int num_anchors;
    int per_cta;
    float high, low;
    int allow_low_quality;
};

__global__ void __launch_bounds__(256) box_iou_match_kernel(const float4* __restrict__ boxes,
                                                            const int* __restrict__ box_offsets,
                                                            int* __restrict__ out_matches, const MatchLaunch L) {
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float4 sbox[kMatchMaxBoxes];
    __shared__ float sarea[kMatchMaxBoxes];
    __shared__ uint32_t best_key[kMatchMaxBoxes];   // read by the other CTAs of the cluster
    __shared__ float best_val[kMatchMaxBoxes];

    // samples are taken longest first (most boxes first), see pick_sample
    static_assert(kMatchMaxBoxes >= kOrderMax, "best_key doubles as the ranking's scratch");
    const int n = pick_sample(box_offsets, reinterpret_cast<int*>(best_key));
    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31;
    const int A = L.num_anchors;
    const int a_base = rank * L.per_cta;
    const int n_local = max(0, min(L.per_cta, A - a_base));     // anchors this CTA owns
    const int b_begin = box_offsets[n];
    const int nb = min(box_offsets[n + 1] - b_begin, kMatchMaxBoxes);
    const int groups = (L.per_cta + kMatchK * T - 1) / (kMatchK * T);   // the same for every CTA of the cluster

    const uint32_t key_m1 = float_key(-1.0f);
    for (int j = tid; j < nb; j += T) {
        const float4 b = boxes[b_begin + j];
        sbox[j] = b;
        sarea[j] = mul_rn(sub_rn(b.w, b.y), sub_rn(b.z, b.x));
        best_key[j] = key_m1;
        best_val[j] = -1.0f;
    }
    __syncthreads();

    if (L.allow_low_quality) {
        for (int g = 0; g < groups; g++) {
            float4 anc[kMatchK];
            float area_a[kMatchK];
            bool valid[kMatchK];
#pragma unroll
            for (int k = 0; k < kMatchK; k++) {
                const int la = (g * kMatchK + k) * T + tid;
                valid[k] = la < n_local;
                anc[k] = valid[k] ? L.anchors[a_base + la] : make_float4(0.f, 0.f, 0.f, 0.f);
                area_a[k] = mul_rn(sub_rn(anc[k].w, anc[k].y), sub_rn(anc[k].z, anc[k].x));
                asm volatile("" : "+f"(area_a[k]));   // opaque from here on: kept in a register, not recomputed per box
            }
            for (int j = 0; j < nb; j++) {
                const float4 b = sbox[j];
                const float area_b = sarea[j];
                float tmax = -1.0f;
#pragma unroll
                for (int k = 0; k < kMatchK; k++) {
                    const float v = iou_ltrb(b, area_b, anc[k], area_a[k]);
                    if (valid[k] && v > tmax) tmax = v;
                }
                const uint32_t kmax = __reduce_max_sync(0xffffffffu, float_key(tmax));
                if (lane == 0 && kmax > key_m1) atomicMax(&best_key[j], kmax);
            }
        }
        __syncthreads();
        cluster.sync();
        for (int j = tid; j < nb; j += T) {
            uint32_t m = key_m1;
#pragma unroll
            for (int r = 0; r < kMatchCluster; r++) m = max(m, *cluster.map_shared_rank(&best_key[j], r));
            best_val[j] = key_float(m);
        }
        __syncthreads();
    }
    // No CTA may leave while another still reads its best_key[]; without low-quality matches this is the only
    // cluster barrier and merely keeps the launch shape uniform.
    cluster.sync();

    int* om = out_matches + (size_t)n * A + a_base;
    for (int g = 0; g < groups; g++) {
        float4 anc[kMatchK];
        float area_a[kMatchK];
        float mval[kMatchK];
        int midx[kMatchK];
        bool lq[kMatchK];
#pragma unroll
        for (int k = 0; k < kMatchK; k++) {
            const int la = (g * kMatchK + k) * T + tid;
            anc[k] = la < n_local ? L.anchors[a_base + la] : make_float4(0.f, 0.f, 0.f, 0.f);
            area_a[k] = mul_rn(sub_rn(anc[k].w, anc[k].y), sub_rn(anc[k].z, anc[k].x));
            asm volatile("" : "+f"(area_a[k]));       // opaque from here on: kept in a register, not recomputed per box
            mval[k] = -1.0f;
            midx[k] = -1;
            lq[k] = false;
        }
        for (int j = 0; j < nb; j++) {
            const float4 b = sbox[j];
            const float area_b = sarea[j];
            const float bj = best_val[j];
#pragma unroll
            for (int k = 0; k < kMatchK; k++) {
                const float v = iou_ltrb(b, area_b, anc[k], area_a[k]);
                if (v > mval[k]) { mval[k] = v; midx[k] = j; }
                // |v - best| < 1e-6 in double == |v - best| <= (float)1e-6 for a float difference
                if (L.allow_low_quality && fabsf(sub_rn(v, bj)) <= 1e-6f) lq[k] = true;
            }
        }
#pragma unroll
        for (int k = 0; k < kMatchK; k++) {
            const int la = (g * kMatchK + k) * T + tid;
            if (la >= n_local) continue;
            int res = midx[k];
            if (!lq[k]) {
                if (mval[k] < L.low) res = -1;
                else if (mval[k] < L.high) res = -2;
            }
            om[la] = res;
        }
    }
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200k_box_iou_match(const float* boxes, const int32_t* box_offsets, int n, int max_boxes_per_sample,
                                    const rb200_box_matcher_params* p, int32_t* out_matches, void* stream_v) {
    if (n == 0) return RB200_OK;
    if (!boxes || !box_offsets || !p || !p->anchors || !out_matches || n < 0 || p->num_anchors <= 0) {
        set_error("rb200k_box_iou_match: null pointer or non-positive size");
        return RB200_E_INVALID;
    }
    if (max_boxes_per_sample < 1 || max_boxes_per_sample > kMatchMaxBoxes) {
        set_error("rb200k_box_iou_match: max_boxes_per_sample %d outside [1,%d]", max_boxes_per_sample, kMatchMaxBoxes);
        return RB200_E_LIMIT;
    }
    if (n > 65535) {
        set_error("rb200k_box_iou_match: batch %d exceeds 65535", n);
        return RB200_E_LIMIT;
    }
    if (((uintptr_t)boxes | (uintptr_t)p->anchors) & 15) {
        set_error("rb200k_box_iou_match: boxes and anchors must be 16-byte aligned");
        return RB200_E_INVALID;
    }
    MatchLaunch L;
    L.anchors = reinterpret_cast<const float4*>(p->anchors);
    L.num_anchors = p->num_anchors;
    L.per_cta = (p->num_anchors + kMatchCluster - 1) / kMatchCluster;
    L.high = p->high_threshold;
    L.low = p->low_threshold;
    L.allow_low_quality = p->allow_low_quality_matches ? 1 : 0;
    int threads = (((L.per_cta + kMatchK - 1) / kMatchK) + 31) & ~31;
    threads = threads < 64 ? 64 : (threads > 256 ? 256 : threads);

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kMatchCluster, (unsigned)n, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = (cudaStream_t)stream_v;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kMatchCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, box_iou_match_kernel, reinterpret_cast<const float4*>(boxes), box_offsets,
                                           out_matches, L),
                        "cudaLaunchKernelEx(box_iou_match_kernel)");
    if (rc) return rc;
    count_launch();
    return RB200_OK;
}
