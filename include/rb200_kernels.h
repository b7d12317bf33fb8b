/*
 * rb200_kernels.h — C ABI of the sm_100a augmentation kernels.
 *
 * Every entry point takes plain device pointers, POD per-sample tables and a CUDA stream
 * (passed as void* so that no CUDA header is needed to bind it). Nothing here allocates
 * unless the comment of the entry point says so. All entry points return 0 on success or a
 * negative RB200_E_* code; rb200k_last_error() returns the text of the last failure on the
 * calling thread.
 *
 * Image convention (as the reference's loader output, rocAL/source/loaders/image/
 * image_read_and_decode.cpp:217-244): uint8, interleaved channels (HWC), 3 channels, one
 * image = `height` rows of `stride` bytes starting `offset` bytes after an arena base. The
 * valid region of every sample starts at pixel (0,0) of its slot unless an ROI says otherwise.
 *
 * Each "replaces" note names the reference code whose work the entry point does. The
 * reference runs these operators as OpenVX nodes of the vx_rpp extension (one node per
 * operator per batch); here one launch handles the whole ragged batch.
 */
#ifndef RB200_KERNELS_H
#define RB200_KERNELS_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef RB200_API
#define RB200_API __attribute__((visibility("default")))
#endif

#define RB200_OK 0
#define RB200_E_INVALID (-1)   /* bad argument (null pointer, size out of range, bad enum) */
#define RB200_E_CUDA (-2)      /* a CUDA runtime call failed; see rb200k_last_error()    */
#define RB200_E_LIMIT (-3)     /* size beyond a documented maximum of the entry point    */

/* Output element types and layouts; numeric values follow RocalTensorOutputType and
 * RocalTensorLayout (rocAL/include/api/rocal_api_types.h:211-232,195-206). */
enum { RB200_FP32 = 0, RB200_FP16 = 1, RB200_UINT8 = 2 };
enum { RB200_NHWC = 0, RB200_NCHW = 1 };

/* ---------------------------------------------------------------------------------------
 * Bilinear resample family: [crop ->] resize(bilinear) [-> crop] [-> mirror] [-> normalize]
 * ------------------------------------------------------------------------------------- */

/* One sample of a resample launch (64 bytes).
 *   roi_*   : rectangle of the source that is resized (whole image for a plain resize; the
 *             crop window for crop->resize chains).
 *   dst_w/h : size of the (virtual) resized image.
 *   crop_*  : window of the resized image that is written to the output; crop_w/crop_h are
 *             the valid output extent of this sample.
 *   mirror  : 1 = output column x shows resized column crop_x + crop_w-1-x.
 */
typedef struct rb200_resample_sample {
    uint64_t src_offset;
    uint32_t src_stride;
    int32_t roi_x, roi_y, roi_w, roi_h;
    int32_t dst_w, dst_h;
    int32_t crop_x, crop_y, crop_w, crop_h;
    int32_t mirror;
    int32_t reserved[2];
} rb200_resample_sample;

/* Launch-wide description of the output tensor and of the arithmetic after interpolation.
 *   out            : device pointer, N samples of out_h*out_w*3 elements each.
 *   out_dtype      : RB200_FP32 / RB200_FP16 / RB200_UINT8.
 *   out_layout     : RB200_NCHW ([N][3][out_h][out_w]) or RB200_NHWC ([N][out_h][out_w][3]).
 *   normalize      : 0 = store the rounded uint8 value of the resized pixel as is;
 *                    1 = store fma(u8, mul[c], add[c]) (for RB200_UINT8: rounded to nearest
 *                        even and saturated).
 *   fill_padding   : 1 = elements outside a sample's crop_w x crop_h are written as 0;
 *                    0 = they are left untouched (the reference leaves them undefined).
 *   interpolation  : RB200_INTERP_BILINEAR (2 x 2 taps) or RB200_INTERP_TRIANGULAR (a triangle
 *                    filter whose support grows with the down-scale ratio: ceil(2*max(ratio,1))
 *                    taps per axis, normalised weights, result truncated to uint8), the
 *                    arithmetic of resize_generic_pln1_hip_tensor
 *                    (rocAL/rocAL_hip/rocal_hip_kernels.cpp:487-589) applied to each channel.
 *                    RB200_INTERP_BICUBIC / _LANCZOS / _GAUSSIAN / _NEAREST run the same skeleton with
 *                    another weight function and base radius B (support = B*max(ratio,1) per side):
 *                    bicubic = Keys' cubic with a = -0.5, B = 2; lanczos = sinc(x)*sinc(x/3), B = 3;
 *                    gaussian = exp(-4 x^2), B = 1; nearest = one tap, B = 0.5. The reference keeps
 *                    these four filters in the RPP library, so their definitions here are this
 *                    library's own (rocal_api_types.h:347-367 only names them).
 */
enum { RB200_INTERP_BILINEAR = 0, RB200_INTERP_TRIANGULAR = 1, RB200_INTERP_BICUBIC = 2, RB200_INTERP_LANCZOS = 3,
       RB200_INTERP_GAUSSIAN = 4, RB200_INTERP_NEAREST = 5 };
/* Kernel choice for bilinear launches. AUTO picks by output width and source span; TILE forces the shared-memory
 * tile kernel where AUTO would stream rows through the bulk-copy ring; withholding h_samples selects the direct
 * (global gather) kernel. The row-streaming kernel has two rings: PAIRS stages the two tap rows of every output row
 * (a source row that two output rows share is fetched twice - an L2 hit in device memory), ROWS stages every distinct
 * source row once (what a source in mapped host memory wants: nothing crosses the link twice). AUTO asks the runtime
 * where `arena` lives and takes ROWS for host memory, PAIRS otherwise; a caller that knows can say so and save the
 * query. All of them compute the same values. */
enum { RB200_RESAMPLE_PATH_AUTO = 0, RB200_RESAMPLE_PATH_TILE = 1, RB200_RESAMPLE_PATH_ROWS = 2, RB200_RESAMPLE_PATH_PAIRS = 3 };
typedef struct rb200_resample_params {
    void* out;
    int32_t out_w, out_h;
    int32_t out_dtype, out_layout;
    int32_t normalize, fill_padding;
    float mul[3];
    float add[3];
    int32_t interpolation;
    int32_t path;                /* RB200_RESAMPLE_PATH_*: which of the bilinear kernels runs; the results are identical */
    int32_t overlap;             /* 1 = this launch may overlap the tail of the kernel enqueued just before it in the
                                    stream, see "Overlapping launches" below; 0 = plain stream order */
    int32_t strip_rows;          /* tuning: output rows per CTA of the row-streaming kernel, 4..32; 0 = chosen by the
                                    library from the grid size and the kernel's occupancy. The results do not depend on it */
    int32_t* status;             /* where a kernel that gives up on a bounded wait writes 1: a 4-byte word the device can
                                    write (device memory, or mapped pinned host memory); NULL = the library-wide word of
                                    this device that rb200k_device_status() reads */
    uint64_t arena_bytes;        /* size of the source arena, 0 = unknown; see "Sizes and the bounds-checking build" */
    uint64_t out_bytes;          /* size of the output buffer, 0 = unknown */
} rb200_resample_params;

/* Resize / ResizeCropMirror / ResizeMirrorNormalize / fused Resize+CropMirrorNormalize.
 * replaces: vxExtRppResize (rocAL/source/augmentations/geometry_augmentations/node_resize.cpp:56),
 *           vxExtRppCropMirrorNormalize (node_crop_mirror_normalize.cpp:87),
 *           vxExtRppResizeCropMirror (node_resize_crop_mirror.cpp:59),
 *           vxExtRppResizeMirrorNormalize (node_resize_mirror_normalize.cpp:90), and the HIP
 *           kernel resize_bilinear_pkd_hip_tensor (rocAL/rocAL_hip/rocal_hip_kernels.cpp:446-485)
 *           whose interpolation arithmetic it follows.
 * `samples` is a DEVICE pointer to n structs; `h_samples` is the same table in HOST memory
 * (used to size the launch; not retained after return).
 */
RB200_API int rb200k_resample(const uint8_t* arena, const rb200_resample_sample* samples,
                    const rb200_resample_sample* h_samples, int n,
                    const rb200_resample_params* params, void* stream);

/* ---------------------------------------------------------------------------------------
 * Pointwise family: crop / flip / colour ops / normalize / layout+dtype conversion
 * ------------------------------------------------------------------------------------- */

enum {
    RB200_COLOR_NONE = 0,        /* copy (crop, flip, CropMirrorNormalize, to_tensor)        */
    RB200_COLOR_BRIGHTNESS = 1,  /* y = alpha*x + beta; a non-zero hue field tilts the offset: beta + hue for
                                    R, beta - hue for B (exposure and colour temperature are this operator)  */
    RB200_COLOR_CONTRAST = 2,    /* y = (x - beta)*alpha + beta  (alpha=factor, beta=center) */
    RB200_COLOR_TWIST = 3,       /* hue/saturation in HSV, then y = alpha*x + beta           */
    RB200_COLOR_GAMMA = 4,       /* y = 255 * (x/255)^alpha                                  */
    RB200_COLOR_BLEND = 5        /* y = alpha*x + (1 - alpha)*x2, x2 = the same pixel of a second source image
                                    at arena + src2_offset (row pitch src2_stride)            */
};

/* One sample of a pointwise launch (64 bytes). The window roi_w x roi_h at (roi_x, roi_y) of
 * the source is written to output (0,0)..(roi_w-1, roi_h-1); flip_h / flip_v reverse the
 * column / row order inside the window. */
typedef struct rb200_pointwise_sample {
    uint64_t src_offset;
    uint32_t src_stride;
    int32_t roi_x, roi_y, roi_w, roi_h;
    int32_t flip_h, flip_v;
    float alpha, beta, hue, sat;
    uint32_t src2_offset_lo, src2_offset_hi;   /* RB200_COLOR_BLEND: 64-bit byte offset of the second source image */
    uint32_t src2_stride;                      /* relative to the arena pointer (wrap-around arithmetic), its pitch */
} rb200_pointwise_sample;

/* Arithmetic of the colour operators on uint8 output.
 *   RB200_ARITH_EXACT  every float operation rounds once, in the order of the CPU restatement the tests compare with:
 *                      results are bit-identical to it.
 *   RB200_ARITH_FAST   the same functions evaluated with fused multiply-adds, one hardware reciprocal and a periodic
 *                      form of the HSV -> RGB step (no table, no wrap-around selects): every output byte is within
 *                      one level of the EXACT result; about twice the ColorTwist / Hue / Saturation throughput.
 *                      Operators other than ColorTwist / Hue / Saturation, and outputs other than uint8 without
 *                      normalisation, run the EXACT code under either setting. */
enum { RB200_ARITH_EXACT = 0, RB200_ARITH_FAST = 1 };
typedef struct rb200_pointwise_params {
    void* out;
    int32_t out_w, out_h;
    int32_t out_dtype, out_layout;
    int32_t color_op;            /* RB200_COLOR_*                                            */
    int32_t normalize, fill_padding;
    int32_t reverse_channels;    /* 1 = output channel c shows source channel 2-c            */
    float mul[3];
    float add[3];
    int32_t arith;               /* RB200_ARITH_EXACT (0) or RB200_ARITH_FAST (1), see below */
    int32_t overlap;             /* as rb200_resample_params.overlap */
    int32_t* status;             /* as rb200_resample_params.status */
    uint64_t arena_bytes;        /* as rb200_resample_params.arena_bytes / out_bytes */
    uint64_t out_bytes;
} rb200_pointwise_params;

/* Crop / Flip / CropMirrorNormalize / Brightness / Contrast / Hue / Saturation / ColorTwist
 * (+ fused Flip) / u8 -> fp32|fp16 NCHW|NHWC conversion.
 * replaces: vxExtRppCrop (node_crop.cpp:47, node_ssd_random_crop.cpp:58), vxExtRppFlip
 *           (node_flip.cpp:44), vxExtRppCropMirrorNormalize (node_crop_mirror_normalize.cpp:87),
 *           vxExtRppBrightness / Contrast / Hue / Saturation / ColorTwist
 *           (color_augmentations/node_*.cpp), the converters Hip_CopyInt8ToNHWC_* /
 *           Hip_CopyInt8ToNCHW_* (rocAL/rocAL_hip/rocal_hip_kernels.cpp:40-217) and the CPU
 *           loop of MasterGraph::to_tensor (rocAL/source/pipeline/master_graph.cpp:672-853).
 */
RB200_API int rb200k_pointwise(const uint8_t* arena, const rb200_pointwise_sample* samples,
                     const rb200_pointwise_sample* h_samples, int n,
                     const rb200_pointwise_params* params, void* stream);

/* ---------------------------------------------------------------------------------------
 * Affine gather family: WarpAffine / Rotate
 * ------------------------------------------------------------------------------------- */

/* One sample (64 bytes). m = {m00, m01, m10, m11, t0, t1} in the packing order of the
 * reference ([x0, y0, x1, y1, o0, o1], node_warp_affine.cpp:43-48). For output pixel (x,y):
 *   dx = x - (float)(out_w/2), dy = y - (float)(out_h/2)                   (integer halves)
 *   sx = m00*dx + m01*dy + t0 + src_w/2.f ;  sy = m10*dx + m11*dy + t1 + src_h/2.f
 * bilinear sample at (sx, sy); a tap position whose floor lies outside the source gives 0. */
typedef struct rb200_warp_sample {
    uint64_t src_offset;
    uint32_t src_stride;
    int32_t src_w, src_h;
    float m[6];
    int32_t dst_w, dst_h;        /* valid output extent of this sample (<= out_w, out_h)     */
    int32_t reserved[3];
} rb200_warp_sample;

typedef struct rb200_warp_params {
    void* out;                   /* uint8 NHWC [N][out_h][out_w][3]                          */
    int32_t out_w, out_h;
    int32_t fill_padding;
    int32_t overlap;             /* as rb200_resample_params.overlap */
    int32_t* status;             /* as rb200_resample_params.status (only the bounds-checking build writes it) */
    uint64_t arena_bytes;        /* as rb200_resample_params.arena_bytes / out_bytes */
    uint64_t out_bytes;
} rb200_warp_params;

/* replaces: vxExtRppWarpAffine (node_warp_affine.cpp:61), vxExtRppRotate (node_rotate.cpp:43). */
RB200_API int rb200k_warp_affine(const uint8_t* arena, const rb200_warp_sample* samples, int n,
                       const rb200_warp_params* params, void* stream);

/* ---------------------------------------------------------------------------------------
 * SSD box encoder
 * ------------------------------------------------------------------------------------- */

typedef struct rb200_box_encoder_params {
    const float* anchors;        /* device, [num_anchors][4] ltrb                            */
    int32_t num_anchors;
    float criteria;
    float means[4];
    float inv_stds[4];           /* (float)(1.0 / stds[i]), evaluated in double              */
    int32_t offset;              /* 1 = offset encoding                                      */
    float scale;
} rb200_box_encoder_params;

/* Matches every anchor of every sample with a ground-truth box and writes the encoded box
 * and label. boxes: device [total][4] ltrb; labels: device [total]; box_offsets: device
 * [n+1] prefix of box counts (sample i owns boxes box_offsets[i] .. box_offsets[i+1]-1; a
 * sample without boxes, which the reference does not define, leaves every anchor unmatched).
 * out_boxes: device [n][num_anchors][4] fp32 (xc,yc,w,h); out_labels: device
 * [n][num_anchors] int32. Tie rules are those of the CPU encoder: the best anchor of a box
 * is the lowest index among equals; the best box of an anchor is the highest index among
 * equals. max_boxes_per_sample must be >= the largest count in the batch (<= 1024);
 * num_anchors <= 65536, n <= 65535. boxes, anchors and out_boxes must be 16-byte aligned.
 * replaces: BoundingBoxGraph::update_box_encoder_meta_data
 *           (rocAL/source/meta_data/bounding_box_graph.cpp:150-220) and BoxEncoderGpu::Run +
 *           BoxEncode<256> (rocAL/rocAL_hip/box_encoder_hip.cpp:123-278).
 */
RB200_API int rb200k_box_encode(const float* boxes, const int32_t* labels, const int32_t* box_offsets,
                      int n, int max_boxes_per_sample, const rb200_box_encoder_params* params,
                      float* out_boxes, int32_t* out_labels, void* stream);

/* Box IoU matcher: out_matches[n][num_anchors] int32 = index (within the sample) of the box with the
 * highest IoU for each anchor, -1 where that IoU is below low_threshold, -2 where it is below
 * high_threshold; with allow_low_quality_matches every anchor whose IoU with some box is within 1e-6
 * of that box's best IoU keeps its match. boxes / box_offsets as for rb200k_box_encode (device
 * pointers, boxes and anchors 16-byte aligned); at most 1024 boxes per sample, any number of anchors.
 * An anchor that no box matches at all (sample without boxes, NaN IoUs) starts from -1.
 * replaces: BoundingBoxGraph::update_box_iou_matcher
 *           (rocAL/source/meta_data/bounding_box_graph.cpp:222-284). */
typedef struct rb200_box_matcher_params {
    const float* anchors;        /* device, [num_anchors][4] ltrb */
    int32_t num_anchors;
    float high_threshold, low_threshold;
    int32_t allow_low_quality_matches;
} rb200_box_matcher_params;

RB200_API int rb200k_box_iou_match(const float* boxes, const int32_t* box_offsets, int n, int max_boxes_per_sample,
                         const rb200_box_matcher_params* params, int32_t* out_matches, void* stream);

/* ---------------------------------------------------------------------------------------
 * Boxes through a crop window and a mirror (metadata of the crop-type operators)
 * ------------------------------------------------------------------------------------- */

/* One sample (32 bytes): the window in the normalised coordinates of the sample's boxes, and whether the boxes are
 * mirrored afterwards (left-right, top-bottom). */
typedef struct rb200_box_window {
    float l, t, r, b;
    int32_t mirror_h, mirror_v;
    int32_t reserved[2];
} rb200_box_window;
enum { RB200_BOX_RULE_QUARTER_AREA = 0, RB200_BOX_RULE_CENTRE = 1 };

/* The box update of the reference's crop-type meta nodes for boxes that already live in device memory (the pipeline
 * transforms its own boxes on the host, where they are fed and where the window samplers need them).
 *   RB200_BOX_RULE_QUARTER_AREA: a box stays when at least a quarter of its area lies in the window
 *     (MetaNode::BBoxIntersectionOverUnion without is_iou, threshold 0.25: meta_node_crop.cpp:59-78,
 *     meta_node_crop_mirror_normalize.cpp:53-90, meta_node_resize_crop_mirror.cpp:66-100); a sample left without boxes
 *     gets the whole window, label 0.
 *   RB200_BOX_RULE_CENTRE: a box stays when its centre lies strictly inside the window (SSD crop and random bbox crop,
 *     bounding_box_graph.cpp:98-110); a sample left without boxes gets one empty box, label 0.
 * Kept boxes are clipped to the window, re-normalised to it, mirrored (meta_node_flip.cpp:40-60) and written in their
 * original order: sample i's boxes at out_boxes[out_offsets[i] .. out_offsets[i + 1]), which makes the three output
 * arrays direct inputs of rb200k_box_encode / rb200k_box_iou_match. All pointers are device pointers; boxes and
 * out_boxes 16-byte aligned; out_boxes / out_labels hold at least (input boxes + n) entries, out_offsets n + 1.
 * Enqueues three small kernels on `stream`. */
RB200_API int rb200k_box_transform(const float* boxes, const int32_t* labels, const int32_t* box_offsets, int n,
                         const rb200_box_window* windows, int rule, float* out_boxes, int32_t* out_labels,
                         int32_t* out_offsets, void* stream);

/* ---------------------------------------------------------------------------------------
 * Normalize / Transpose (neighbouring operators of the augmentation path)
 * ------------------------------------------------------------------------------------- */

/* Mean / standard-deviation normalisation of uint8 HWC images:  out = scale * (x - mean) / stddev + shift, float32 or
 * float16, same layout (NHWC, [N][out_h][out_w][3], the sample's window at the origin). axis_mask names the axes that
 * are reduced when mean and / or stddev are computed from the data: bit 0 = height, bit 1 = width, bit 2 = channel
 * (the reference's convention for an NHWC tensor, node_normalize.cpp:42-50); the statistics then have one value per
 * index of the remaining axes - mask 3 gives one mean per channel, mask 7 one per image, mask 1 one per column and
 * channel. Given values (compute_* = 0) are per-channel constants. Computed statistics are those of the whole
 * population (divisor = number of values); a zero standard deviation yields out = shift.
 *
 * The statistics are accumulated exactly (integer sums of x and x^2, 64-bit atomics) in `scratch`: device memory of at
 * least rb200k_normalize_scratch_bytes(n, max_w, max_h, axis_mask) bytes that the caller owns; it needs no
 * initialisation (the call clears what it uses) and holds nothing of value afterwards. With neither statistic
 * computed no scratch is needed (NULL is accepted). The call enqueues a clear, the sums, a small finishing kernel and the
 * element-wise pass on `stream`.
 * replaces: vxExtRppNormalize (rocAL/source/augmentations/effects_augmentations/node_normalize.cpp:105),
 *           rocalNormalize (rocAL/include/api/rocal_api_augmentation.h:1294). The arithmetic lives in RPP; the
 *           definitions above are this library's reading of the documented formula (rocAL_pybind/amd/rocal/fn.py:1216-1223). */
typedef struct rb200_normalize_params {
    void* out;
    int32_t out_w, out_h;
    int32_t out_dtype;           /* RB200_FP32 or RB200_FP16 */
    int32_t axis_mask;           /* 1..7 when a statistic is computed */
    int32_t compute_mean, compute_stddev;
    int32_t fill_padding;        /* 1 = elements outside a sample's window are written as 0 */
    float mean[3], stddev[3];    /* per-channel values for the statistic(s) that are not computed */
    float scale, shift;
    uint64_t arena_bytes;        /* as rb200_resample_params.arena_bytes / out_bytes; trouble goes to the library-wide */
    uint64_t out_bytes;          /* status word */
} rb200_normalize_params;

RB200_API size_t rb200k_normalize_scratch_bytes(int n, int max_w, int max_h, int axis_mask);
RB200_API int rb200k_normalize(const uint8_t* arena, const rb200_pointwise_sample* samples,
                     const rb200_pointwise_sample* h_samples, int n, const rb200_normalize_params* params,
                     void* scratch, size_t scratch_bytes, void* stream);

/* rb200k_normalize without a scratch argument: the statistics are accumulated in a fixed 1 MiB array that is part of
 * the library itself (65 536 slots of 16 bytes; every GPU that loads the library holds it until the process exits).
 * The entry point has no counterpart in the reference. It is for callers that cannot hand rb200k_normalize a scratch
 * buffer: a host program that binds this C ABI from a language without a CUDA binding of its own (cgo, JNI, ctypes)
 * has no way to create device memory, and a loader that runs beside a framework whose allocator has already claimed
 * the whole device may find that an allocation of its own fails or stalls. Nothing is allocated here or further down:
 * no cudaMalloc, no cudaFree, no allocating library routine; the call enqueues a clear of the slots it uses, the same
 * kernels as rb200k_normalize, and returns.
 *   limit   n x (statistics per sample) <= 65 536, where the statistics per sample follow axis_mask and the OUTPUT
 *           size: 3 (mask 3), 1 (mask 7), 3*out_w (mask 1), 3*out_h (mask 2), out_w (5), out_h (6), out_w*out_h (4).
 *           A larger batch is refused with RB200_E_LIMIT and a message that names both numbers. When neither statistic
 *           is computed the array is not touched and no limit applies.
 *   set-up  the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *           current) and keeps it; make that first call before any stream capture is started on the device. Devices
 *           0..63 are supported.
 *   sharing every call on a device uses the same array, and the array keeps what the last call left in it (each call
 *           clears the slots it is about to use). Two calls whose GPU work can overlap - different streams, or
 *           different host threads - race on it and corrupt each other's statistics: issue them on one stream, or
 *           order them with events.
 * Results are identical to rb200k_normalize's. */
RB200_API int rb200k_normalize_static(const uint8_t* arena, const rb200_pointwise_sample* samples,
                            const rb200_pointwise_sample* h_samples, int n, const rb200_normalize_params* params,
                            void* stream);

/* Axis permutation of uint8 HWC images: sample i's window, d = (h, w, 3), becomes an array of extents
 * (d[perm[0]], d[perm[1]], d[perm[2]]) at the origin of its slot out[i][out_dims[0]][out_dims[1]][out_dims[2]] (the
 * maximum shape of the output tensor, the reference's padded-tensor convention); elements of the slot outside the
 * sample's extents are left untouched, a window larger than the slot is clipped. flip_* of the sample table are
 * ignored.
 * replaces: vxExtRppTranspose, rocalTranspose (rocAL/include/api/rocal_api_augmentation.h:1338). */
RB200_API int rb200k_transpose(const uint8_t* arena, const rb200_pointwise_sample* samples, int n, const int32_t perm[3],
                     uint8_t* out, const int32_t out_dims[3], void* stream);

/* ---------------------------------------------------------------------------------------
 * Overlapping launches
 * ------------------------------------------------------------------------------------- */

/* The row-streaming resample kernel, the pointwise vector kernel and the affine kernel are launched with
 * programmatic stream serialization: behind another kernel of the same stream their CTAs may become resident while
 * that kernel's last CTAs still run. With overlap = 0 they then wait, before they touch global memory, until the
 * preceding kernel has completed and its writes are visible - the result is that of a plain in-order launch and only
 * the launch gap is saved. overlap = 1 states that the launch is independent of the kernel enqueued just before it:
 * it reads nothing that kernel writes (images, tables) and writes nothing that kernel reads or writes. Its CTAs then
 * start working at once, which hides the ramp-up and tail of small batches, and wait for the preceding kernel only
 * before they exit, so that completion of this launch still implies completion of everything before it in the
 * stream. Batches of a device-resident loop that use separate input and output buffers qualify; a step that reads
 * the previous step's output does not. Behind a copy or an event wait the launch is an ordinary one either way. */

/* ---------------------------------------------------------------------------------------
 * Bounded waits
 * ------------------------------------------------------------------------------------- */

/* The row-streaming resample kernel and the pointwise vector kernel wait on mbarriers for their bulk copies. Every
 * such wait gives up after a limit (about a second of SM clock): the kernel then writes 1 to its status word, waits
 * (bounded again) for the copies it may still have in flight, and returns with its output incomplete; the context
 * stays usable. The two entries below run the same launches with a caller-chosen limit (SM clock cycles) and, for
 * self-tests, with the producer told not to issue the copies from one row on (skip_row, counted over the source rows a
 * CTA fetches for its strip or tile; -1 = issue everything), so that the give-up path can be exercised without any faulting or endless wait: the
 * skipped copy never starts, so nothing is left in flight. */
RB200_API int rb200k_resample_probe(const uint8_t* arena, const rb200_resample_sample* samples,
                          const rb200_resample_sample* h_samples, int n, const rb200_resample_params* params,
                          void* stream, uint64_t wait_cycles, int skip_row);
RB200_API int rb200k_pointwise_probe(const uint8_t* arena, const rb200_pointwise_sample* samples,
                           const rb200_pointwise_sample* h_samples, int n, const rb200_pointwise_params* params,
                           void* stream, uint64_t wait_cycles, int skip_row);

/* ---------------------------------------------------------------------------------------
 * Sizes and the bounds-checking build
 * ------------------------------------------------------------------------------------- */

/* The source arena. Every sample table addresses its image as arena + src_offset with a row pitch of src_stride
 * bytes. The staging copies fetch whole 16-byte granules (by address), so a launch may read from the granule that
 * holds the first byte of a sample's source rectangle to the end of the granule that holds its last byte: an arena
 * whose images end within 15 bytes of an allocation that is not a multiple of 16 bytes long must be padded. Device and
 * pinned host allocations are far coarser than that, so only sub-allocated arenas need care.
 *
 * out_bytes (resample, pointwise, warp, normalize parameter blocks): when non-zero, every build refuses, with
 * RB200_E_INVALID and before anything is launched, a call whose dense output (n x out_h x out_w x 3 elements) does not
 * fit. The kernels store nowhere else.
 *
 * arena_bytes: when non-zero, the BOUNDS-CHECKING BUILD of the library (`python -m rocal_b200.build --debug-bounds`,
 * librocal_b200_bounds.so; rb200k_version() ends in "+bounds") checks, inside the kernels, each sample's source
 * rectangle as its table row describes it, and every staging copy it issues, against [arena, arena + arena_bytes)
 * widened to whole granules. A sample or a copy that fails is not read: the kernel writes 2 to the launch's status
 * word (see "Bounded waits" for where that word lives), leaves that sample's output unwritten or incomplete, and
 * returns normally; nothing traps and the context stays usable. The release build ignores the field and performs no
 * such checks. rb200k_transpose and the box kernels take no sizes and are not covered. */

/* ---------------------------------------------------------------------------------------
 * Misc
 * ------------------------------------------------------------------------------------- */

/* The library-wide status word of the current device, read and cleared: 0 = fine; 1 = a kernel launched without a
 * status pointer of its own gave up on one of its bounded waits (a copy that never completed) since the last call, its
 * output is then incomplete; 2 = (bounds-checking build) a kernel found a sample or a copy outside the arena and did
 * not read it; -1 = the query itself failed. Synchronises with the device. */
RB200_API int rb200k_device_status(void);

/* Text of the last error on the calling thread ("" if none). */
RB200_API const char* rb200k_last_error(void);

/* Number of kernel launches issued through this library by the calling process so far. */
RB200_API uint64_t rb200k_launch_count(void);

/* Build identification: "rocal_b200 <version> sm_100a", with "+bounds" appended by the bounds-checking build. */
RB200_API const char* rb200k_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RB200_KERNELS_H */
