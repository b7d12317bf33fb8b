/*
 * rb200.h — plain C ABI of the augmentation pipeline (handles, ints, pointers and sizes only).
 *
 * This is what a foreign-function binding (ctypes, cgo, JNI, N-API ...) attaches to. Every
 * function is the C-callable twin of one rocAL API call declared in rocal_api.h (named in its
 * comment, with the reference declaration it replaces), or an extension marked [extension]:
 * something the benchmark configurations need and the reference API cannot express.
 *
 * Status-returning functions give 0 (ROCAL_OK) or a RocalStatus value; handle-returning
 * functions give NULL on failure. The failure text is kept per context:
 * rb200_get_error_message(). No function throws.
 */
#ifndef RB200_H
#define RB200_H

#include <stddef.h>
#include <stdint.h>

#include "rb200_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void* rb200_context; /* RocalContext */
typedef void* rb200_tensor;  /* RocalTensor (rocalTensor*) */
typedef void* rb200_param;   /* RocalIntParam / RocalFloatParam */

/* ---- life cycle: rocalCreate / rocalVerify / rocalRun / rocalRelease (rocal_api.h:83-110) ---- */
RB200_API rb200_context rb200_create(size_t batch_size, int affinity, int gpu_id, size_t cpu_thread_count,
                                     size_t prefetch_queue_depth, int output_tensor_data_type);
RB200_API int rb200_verify(rb200_context ctx);
RB200_API int rb200_run(rb200_context ctx);
RB200_API int rb200_release(rb200_context ctx);
/* rocalGetStatus / rocalGetErrorMessage / rocalGetTimingInfo (rocal_api_info.h:90-106); timing = 4 values in us */
RB200_API int rb200_get_status(rb200_context ctx);
RB200_API const char* rb200_get_error_message(rb200_context ctx);
RB200_API void rb200_get_timing(rb200_context ctx, unsigned long long out_load_decode_process_transfer[4]);
/* [extension] Device time per launch. The reference times its stages on the host (TimingDbg,
 * include/pipeline/timing_debug.h:36-100); with profiling on, this pipeline also brackets the upload and every kernel
 * launch of a batch with CUDA events on its stream and adds the elapsed device times up when the batch is returned by
 * rb200_run. Choose before rb200_verify; RB200_PROFILE=1 in the environment turns it on for every context. Off by
 * default (an event record per launch on the loader thread). rb200_get_step_timing writes up to `capacity` entries -
 * "upload" first, then one per launch of the plan in order - and returns the number of entries there are.
 * The pipeline also marks its stages as NVTX ranges ("rb200 tables", "rb200 upload", "rb200 decode", "rb200 launches")
 * for timeline tools, and RB200_LOG_LEVEL (0 silent, 1 errors - the default, 2 plan at verify and a timing summary at
 * release) controls what it writes to stderr. */
typedef struct rb200_step_timing {
    char name[32];               /* "upload", "resample", "pointwise", "warp_affine", "normalize", "transpose" */
    double gpu_us;               /* device time accumulated over `batches` batches */
    unsigned long long batches;
} rb200_step_timing;
RB200_API int rb200_set_profiling(rb200_context ctx, int on);
RB200_API size_t rb200_get_step_timing(rb200_context ctx, rb200_step_timing* out, size_t capacity);
/* rocalGetRemainingImages / rocalIsEmpty (rocal_api_info.h:66-74): fed but not yet returned samples */
RB200_API size_t rb200_get_remaining_images(rb200_context ctx);
/* Extensions without a reference counterpart: how host-resident source pixels reach the kernels.
 *   RB200_UPLOAD_WHOLE      every image is copied to the device whole;
 *   RB200_UPLOAD_FOOTPRINT  one strided copy per image of the rectangle the batch's kernels can read
 *                           (the crop window mapped back through the resize);
 *   RB200_UPLOAD_ZERO_COPY  (default) a batch fed with rb200_feed_ragged from RB200_MEM_HOST_PINNED memory
 *                           that one resample or pointwise step consumes is not copied: the kernel's bulk
 *                           copies read the rows it needs from the pinned buffer, which must stay valid and
 *                           unchanged until rb200_run has returned that batch. Other batches fall back to
 *                           RB200_UPLOAD_FOOTPRINT.
 * rb200_get_h2d_bytes returns the bytes that have crossed to the device for the context so far (pixels -
 * in zero-copy mode the footprint rectangles - plus per-sample tables and boxes). */
enum { RB200_UPLOAD_WHOLE = 0, RB200_UPLOAD_FOOTPRINT = 1, RB200_UPLOAD_ZERO_COPY = 2 };
RB200_API unsigned long long rb200_get_h2d_bytes(rb200_context ctx);
RB200_API int rb200_set_upload_mode(rb200_context ctx, int mode);

/* [extension] Arithmetic of the colour operators for the batches fed from now on: 0 = RB200_ARITH_EXACT (default;
 * bit-identical to the CPU restatement), 1 = RB200_ARITH_FAST (every uint8 output within one level of EXACT,
 * about twice the ColorTwist / Hue / Saturation throughput); see rb200_kernels.h. Call between rocalVerify and the
 * feed of the first batch it should apply to. Returns 0, or -1 for a bad handle or mode. */
RB200_API int rb200_set_arithmetic(rb200_context ctx, int mode);

/* [extension] Stream hand-off for zero-copy consumers. The output tensors of the batch that rb200_run returned alias
 * ring buffers that go back to the pipeline at the next rb200_run (the reference's rule, master_graph.cpp:928-938);
 * the reference's PyTorch plugin copies them synchronously first (rocAL_pybind/amd/rocal/plugin/pytorch.py:118-143).
 * A consumer that instead reads them in place on its own CUDA stream calls this before the next rb200_run with that
 * stream (a cudaStream_t; NULL = the legacy default stream): the pipeline records an event there and makes its own
 * streams wait for it before the buffers are written again. No host synchronisation takes place. Returns 0 / -1. */
RB200_API int rb200_consumer_fence(rb200_context ctx, void* cuda_stream);

/* [test hook] Self-test of the bounded waits: while wait_cycles is non-zero, the resample and pointwise launches of
 * the batches fed from now on go through rb200k_resample_probe / rb200k_pointwise_probe with that wait limit (SM
 * clock cycles) and skip_row (see rb200_kernels.h); rb200_run then reports the batch as failed
 * (ROCAL_RUNTIME_ERROR, message in rb200_get_error_message) instead of handing out incomplete outputs, and the
 * context stays usable. wait_cycles = 0 switches the probe off. */
RB200_API int rb200_set_wait_probe(rb200_context ctx, unsigned long long wait_cycles, int skip_row);

/* ---- parameters (rocal_api_parameters.h:39-161) ---- */
RB200_API void rb200_set_seed(unsigned seed);
RB200_API unsigned rb200_get_seed(void);
RB200_API rb200_param rb200_create_int_uniform_rand(int start, int end);
RB200_API rb200_param rb200_create_float_uniform_rand(float start, float end);
RB200_API rb200_param rb200_create_int_rand(const int* values, const double* frequencies, unsigned size);
RB200_API rb200_param rb200_create_float_rand(const float* values, const double* frequencies, unsigned size);
RB200_API rb200_param rb200_create_int_parameter(int value);
RB200_API rb200_param rb200_create_float_parameter(float value);
RB200_API int rb200_update_int_parameter(int value, rb200_param p);
RB200_API int rb200_update_float_parameter(float value, rb200_param p);
RB200_API int rb200_update_int_uniform_rand(int start, int end, rb200_param p);
RB200_API int rb200_update_float_uniform_rand(float start, float end, rb200_param p);
RB200_API int rb200_get_int_value(rb200_param p);
RB200_API float rb200_get_float_value(rb200_param p);

/* ---- input ---- */
/* rocalJpegExternalFileSource (rocal_api_data_loaders.h:961-970) in its three modes:
 * ROCAL_EXTSOURCE_RAW_UNCOMPRESSED (decoded pixels), ROCAL_EXTSOURCE_RAW_COMPRESSED (JPEG streams) and
 * ROCAL_EXTSOURCE_FNAME (JPEG files). JPEG input is decoded on the GPU by NVIDIA's nvJPEG library straight into
 * the packed arena the kernels read; max_width x max_height bounds the decoded size. */
RB200_API rb200_tensor rb200_external_source(rb200_context ctx, int color_format, int is_output, unsigned max_width,
                                             unsigned max_height, int external_source_mode);
/* rocalExternalSourceFeedInput (rocal_api_data_transfer.h:101-105): n buffers of max_height x max_width x
 * channels bytes, roi_xywh = 4*n unsigned; in ROCAL_EXTSOURCE_RAW_COMPRESSED mode buffer i is a JPEG stream
 * whose byte length is roi_xywh[4*i+3] (image_read_and_decode.cpp:123-124). The buffers must stay valid until
 * the batch has been returned by rb200_run (the reference queues the pointers too:
 * external_source_reader.cpp:220-233). */
RB200_API int rb200_feed_input(rb200_context ctx, const unsigned char* const* buffers, const unsigned* roi_xywh,
                               size_t n, unsigned max_width, unsigned max_height, unsigned channels, int mode,
                               int layout, int eos);

/* One image of a ragged batch: tightly packed, rows `stride` bytes apart. */
typedef struct rb200_image_desc {
    uint64_t offset; /* of pixel (0,0) from the arena base, bytes */
    uint32_t stride;
    uint32_t width, height;
} rb200_image_desc;
enum { RB200_MEM_HOST = 0, RB200_MEM_HOST_PINNED = 1, RB200_MEM_DEVICE = 2 };
/* [extension] Feeds one batch as a single arena + per-image descriptors instead of n max-size slots
 * (which would move 3-4x the bytes for variable-size images). mem_kind says where the arena lives;
 * a device arena is used in place (no copy), a host arena is uploaded with one asynchronous copy.
 * The arena must stay valid until the batch has been returned by rb200_run.
 * Reads reach the whole 16-byte granules (by address) that enclose each image's rows: device and pinned allocations
 * cover that by themselves; an arena carved out of a larger buffer of the caller's should start on a 16-byte boundary
 * and leave 15 readable bytes after its last image (nothing is ever written there, and an aligned 16-byte read never
 * crosses a page, so a tighter arena cannot fault - it is merely read a few bytes beyond its ends).
 * A RB200_MEM_DEVICE arena is read by the pipeline's own stream without any ordering against the stream that filled it:
 * complete that work (an event the caller waits on, or a stream synchronisation) before feeding. */
RB200_API int rb200_feed_ragged(rb200_context ctx, const void* arena, size_t arena_bytes,
                                const rb200_image_desc* descs, size_t n, int mem_kind);
/* [extension] JPEG streams with their lengths as size_t (same lifetime rule as rb200_feed_input), and JPEG
 * files by name (read at feed time; the FNAME mode of rocalExternalSourceFeedInput). */
RB200_API int rb200_feed_encoded(rb200_context ctx, const unsigned char* const* buffers, const size_t* sizes, size_t n);
RB200_API int rb200_feed_files(rb200_context ctx, const char* const* paths, size_t n);

/* rocalJpegFileSourceSingleShard + rocalCreateLabelReader (rocal_api_data_loaders.h:80-90,
 * rocal_api_meta_data.h:43): a folder of JPEG files (one sub-folder per class, numbered in sorted order; a
 * flat folder is class 0), shard shard_id of shard_count, read and decoded by the context itself - rb200_run
 * needs no feed call. last_batch_policy: 0 fill, 1 drop, 2 partial (rocal_api_types.h:455-495).
 * rocalResetLoaders, rocalGetImageLabels, rocalGetImageNameLen / rocalGetImageName (concatenated names of the
 * current batch, no separators), rocalGetLastBatchPaddedSize. */
/* rocalCreateLabelReader(file_list_path) / rocalCreateTextFileBasedLabelReader: the folder source created next reads the
 * files named in this list ("file_name label" per line, names relative to its source_path) instead of scanning. */
RB200_API int rb200_set_file_list(rb200_context ctx, const char* file_list_path);
RB200_API rb200_tensor rb200_jpeg_file_source(rb200_context ctx, const char* source_path, int color_format, unsigned shard_id,
                                              unsigned shard_count, int is_output, int shuffle, int loop, unsigned max_width,
                                              unsigned max_height, int last_batch_policy, int pad_last_batch_repeated);
/* rocalJpegCOCOFileSourceSingleShard + rocalCreateCOCOReader (rocal_api_data_loaders.h:257-269,
 * rocal_api_meta_data.h:89): images named in a COCO annotation file, looked up under source_path, with their boxes
 * (bbox [x,y,w,h] -> normalized ltrb) and labels (categories renumbered 1.. in file order unless
 * avoid_class_remapping); the boxes follow the graph's crops and mirrors and feed the box encoder / matcher. */
RB200_API rb200_tensor rb200_coco_file_source(rb200_context ctx, const char* source_path, const char* json_path, int color_format,
                                              unsigned shard_id, unsigned shard_count, int is_output, int shuffle, int loop,
                                              unsigned max_width, unsigned max_height, int last_batch_policy,
                                              int pad_last_batch_repeated, int avoid_class_remapping);
RB200_API int rb200_reset_loaders(rb200_context ctx);
RB200_API int rb200_get_image_labels(rb200_context ctx, int* labels);
RB200_API unsigned rb200_get_image_name_len(rb200_context ctx, int* lengths);
RB200_API int rb200_get_image_name(rb200_context ctx, char* buf);
RB200_API size_t rb200_get_last_batch_padded_size(rb200_context ctx);
/* rocalGetOneHotImageLabels (label k > 0 sets position k-1, label 0 the last position; int32 [batch][num_classes],
 * output_mem_type 0 = host, 1 = device) and rocalGetImageSizes (width, height of every source image as read; a fused JPEG crop does not change it). */
RB200_API int rb200_get_one_hot_image_labels(rb200_context ctx, void* buf, int num_classes, int output_mem_type);
RB200_API int rb200_get_image_sizes(rb200_context ctx, int* width_height_pairs);
/* rocalGetImageId: the annotation file's "id" of every image of the batch (COCO source only). */
RB200_API int rb200_get_image_ids(rb200_context ctx, int* ids);
/* rocalGetROIImageSizes: width, height of the valid region of every sample after ResizeMirrorNormalize (of the first
 * output when the graph has no such operator). */
RB200_API int rb200_get_roi_image_sizes(rb200_context ctx, int* width_height_pairs);
/* rocalFusedJpegCropSingleShard (rocal_api_data_loaders.h:493-506; decoders.image_slice and
 * decoders.image_random_crop of the Python API): the folder source of rb200_jpeg_file_source whose images reach
 * the graph cut to a random-resized-crop window: area_factor[2] = {min, max} fraction of the image area,
 * aspect_ratio[2] = {min, max} width / height, num_attempts draws before the clamped fallback
 * (RocalRandomCropDecParam, parameter_random_crop_decoder.cpp:41-101). The image is decoded whole; the window is a
 * view into it, so the crop costs no pass over the pixels. The batch seeds come from the context's seed
 * (the reference draws them from std::random_device). */
RB200_API rb200_tensor rb200_fused_jpeg_crop_file_source(rb200_context ctx, const char* source_path, int color_format,
                                                         unsigned shard_id, unsigned shard_count, int is_output,
                                                         const float* area_factor, const float* aspect_ratio, unsigned num_attempts,
                                                         int shuffle, int loop, unsigned max_width, unsigned max_height,
                                                         int last_batch_policy, int pad_last_batch_repeated);
/* [extension] The same windows for an external source fed with encoded JPEG (rb200_feed_encoded / rb200_feed_files);
 * call after rb200_external_source and before rb200_verify. */
RB200_API int rb200_set_random_crop_decoder(rb200_context ctx, const float* area_factor, const float* aspect_ratio,
                                            unsigned num_attempts);
/* [extension] Windows {x, y, w, h} of the current batch inside the decoded images, and the batch seed they came from
 * (either pointer may be null). */
RB200_API int rb200_get_decoder_crop_windows(rb200_context ctx, unsigned* xywh, unsigned* batch_seed);
/* [extension] Host only, no context: the n windows that batch seed `batch_seed` gives images of
 * shapes_hw[n][2] = {height, width}. */
RB200_API int rb200_random_crop_windows(unsigned batch_seed, const int* shapes_hw, size_t n, const float* area_factor,
                                        const float* aspect_ratio, unsigned num_attempts, unsigned* out_xywh);
/* rocalRandomBBoxCrop (rocal_api_meta_data.h:245; fn.random_bbox_crop): every source image of a batch reaches the graph
 * cut to a window sampled around its boxes, and the boxes follow the window (a box is kept when its centre lies strictly
 * inside; kept boxes are clipped and re-normalised to the window). The window of a sample: one of seven minimum-IoU
 * options {-1, 0.1, 0.3, 0.5, 0.7, 0.9, whole image}; width and height factors in 0.3 .. 1 with a ratio in 0.5 .. 2; left
 * edge aligned to 8 pixels; with all_boxes_overlap every box must reach the option's IoU with the window; one box centre
 * must lie inside; a failed draw starts over (RandomBBoxCropReader::get_batch_crop_coords,
 * source/meta_data/randombboxcrop_reader.cpp:216-313). has_shape != 0 keeps the whole image, as there. The window is a
 * view into the source (only its pixels are uploaded), so the crop costs no pass of its own. The arguments the
 * reference accepts and never reads (no_crop, aspect_ratio, crop size, num_attempts, scaling, total_num_attempts) are
 * taken by the rocalRandomBBoxCrop shim and dropped. seed starts the 128 per-position generators, which the reference
 * seeds from std::random_device. Call after the source and before rb200_verify; the batches must carry boxes
 * (rb200_feed_boxes or a COCO source). */
RB200_API int rb200_random_bbox_crop(rb200_context ctx, int all_boxes_overlap, int has_shape, unsigned seed);
/* [extension] The windows of the current batch as sampled: n x {x, y, w, h} as fractions of the image. The pixel
 * windows are what rb200_get_decoder_crop_windows returns. */
RB200_API int rb200_get_bbox_crop_windows(rb200_context ctx, float* xywh);
/* [extension] Host only, no context: the windows a fresh sampler gives n samples in turn. boxes_ltrb holds
 * box_offsets[n] boxes normalized to their image, sample i owning boxes box_offsets[i] .. box_offsets[i + 1] - 1;
 * img_widths[n] in pixels (for the 8-pixel alignment). */
RB200_API int rb200_bbox_crop_windows(unsigned seed, int all_boxes_overlap, int has_shape, const float* boxes_ltrb,
                                      const int* box_offsets, size_t n, const int* img_widths, float* out_xywh);
/* [extension] Ground-truth boxes of the next fed batch: normalized ltrb, labels, counts[n]. The reference
 * can attach boxes only through a dataset reader keyed by file name (master_graph.cpp:983-984). */
RB200_API int rb200_feed_boxes(rb200_context ctx, const float* ltrb, const int* labels, const int* counts, size_t n);
/* [extension] Per-sample crop anchors in [0,1] for the next batch of a CropMirrorNormalize output
 * (the reference's start_x/start_y are one scalar pair for the whole batch). */
RB200_API int rb200_set_crop_anchors(rb200_context ctx, rb200_tensor cmn_output, const float* anchor_x,
                                     const float* anchor_y, size_t n);
/* [extension] Per-sample affine tables [n][6] = {x0,y0,x1,y1,o0,o1} for the next batch of a WarpAffine
 * output (the reference draws the six coefficients independently, node_warp_affine.cpp:92-101). */
RB200_API int rb200_set_affine(rb200_context ctx, rb200_tensor warp_output, const float* m6, size_t n);

/* ---- augmentations: same arguments as the rocal* calls of rocal_api.h, std::vector flattened ---- */
RB200_API rb200_tensor rb200_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                    int is_output, int scaling_mode, unsigned max_w, unsigned max_h,
                                    unsigned resize_shorter, unsigned resize_longer, int interpolation,
                                    int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_resize_mirror_normalize(rb200_context ctx, rb200_tensor in, unsigned dest_width,
                                                     unsigned dest_height, const float* mean, const float* std_dev,
                                                     size_t n_mean, int is_output, int scaling_mode, unsigned max_w,
                                                     unsigned max_h, unsigned resize_shorter, unsigned resize_longer,
                                                     int interpolation, rb200_param mirror, int out_layout,
                                                     int out_dtype);
RB200_API rb200_tensor rb200_crop_mirror_normalize(rb200_context ctx, rb200_tensor in, unsigned crop_height,
                                                   unsigned crop_width, float start_x, float start_y,
                                                   const float* mean, const float* std_dev, size_t n_mean,
                                                   int is_output, rb200_param mirror, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_crop(rb200_context ctx, rb200_tensor in, int is_output, rb200_param crop_width,
                                  rb200_param crop_height, rb200_param crop_pos_x, rb200_param crop_pos_y,
                                  int out_layout, int out_dtype);
/* rocalRandomCrop, rocalCropResize, rocalCropResizeFixed, rocalROIResize (rocal_api_augmentation.h): windows of
 * RocalRandomCropParam (up to five area / aspect draws for a window strictly inside the image, else the central crop
 * clamped to aspect 0.75..1.333; parameter_random_crop.cpp:48-97) - cut out (RandomCrop) or stretched to
 * dest_width x dest_height in the same launch (CropResize); ROIResize stretches the fixed window roi_w x roi_h at
 * (roi_pos_x, roi_pos_y). Null parameters take the reference's default ranges. */
/* [extension] Host only, no context: the random-area windows {x, y, w, h} for n images of wh[n][2] = {width, height},
 * drawn from the given parameters in sample order (what rb200_random_crop / rb200_crop_resize do per batch). */
RB200_API int rb200_random_area_windows(const unsigned* wh, size_t n, rb200_param area, rb200_param aspect_ratio,
                                        rb200_param x_drift, rb200_param y_drift, unsigned* out_xywh);
RB200_API rb200_tensor rb200_random_crop(rb200_context ctx, rb200_tensor in, int is_output, rb200_param crop_area_factor,
                                         rb200_param crop_aspect_ratio, rb200_param crop_pos_x, rb200_param crop_pos_y,
                                         int num_of_attempts, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_crop_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                         int is_output, rb200_param area, rb200_param aspect_ratio, rb200_param x_center_drift,
                                         rb200_param y_center_drift, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_crop_resize_fixed(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height,
                                               int is_output, float area, float aspect_ratio, float x_center_drift,
                                               float y_center_drift, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_roi_resize(rb200_context ctx, rb200_tensor in, unsigned dest_width, unsigned dest_height, int is_output,
                                        unsigned roi_h, unsigned roi_w, float roi_pos_x, float roi_pos_y, int interpolation,
                                        int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_crop_fixed(rb200_context ctx, rb200_tensor in, unsigned crop_width, unsigned crop_height,
                                        int is_output, float crop_pos_x, float crop_pos_y, int out_layout,
                                        int out_dtype);
RB200_API rb200_tensor rb200_crop_center_fixed(rb200_context ctx, rb200_tensor in, unsigned crop_width,
                                               unsigned crop_height, int is_output, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_resize_crop_mirror_fixed(rb200_context ctx, rb200_tensor in, unsigned dest_width,
                                                      unsigned dest_height, int is_output, unsigned crop_h,
                                                      unsigned crop_w, rb200_param mirror, int out_layout,
                                                      int out_dtype);
RB200_API rb200_tensor rb200_resize_crop_mirror(rb200_context ctx, rb200_tensor in, unsigned dest_width,
                                                unsigned dest_height, int is_output, rb200_param crop_height,
                                                rb200_param crop_width, rb200_param mirror, int out_layout,
                                                int out_dtype);
RB200_API rb200_tensor rb200_ssd_random_crop(rb200_context ctx, rb200_tensor in, int is_output, int num_of_attempts,
                                             int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_flip(rb200_context ctx, rb200_tensor in, int is_output, rb200_param horizontal,
                                  rb200_param vertical, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_brightness(rb200_context ctx, rb200_tensor in, int is_output, rb200_param alpha,
                                        rb200_param beta, int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_contrast(rb200_context ctx, rb200_tensor in, int is_output, rb200_param factor,
                                      rb200_param center, int out_layout, int out_dtype);
/* rocalExposure (x * 2^factor), rocalGamma (255 * (x/255)^gamma), rocalColorTemp (R + adjustment, B - adjustment; an
 * integer parameter). Null parameters take the reference's default ranges. */
RB200_API rb200_tensor rb200_exposure(rb200_context ctx, rb200_tensor in, int is_output, rb200_param exposure_factor,
                                      int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_gamma(rb200_context ctx, rb200_tensor in, int is_output, rb200_param gamma, int out_layout,
                                   int out_dtype);
RB200_API rb200_tensor rb200_color_temp(rb200_context ctx, rb200_tensor in, int is_output, rb200_param adjustment,
                                        int out_layout, int out_dtype);
/* rocalBlend: in*ratio + in2*(1 - ratio) per pixel, rounded; both inputs have the same maximum size. */
RB200_API rb200_tensor rb200_blend(rb200_context ctx, rb200_tensor in, rb200_tensor in2, int is_output, rb200_param ratio,
                                   int out_layout, int out_dtype);
/* rocalNormalize (rocAL/include/api/rocal_api_augmentation.h:1294): out = scale * (x - mean) / std_dev + shift on the
 * uint8 NHWC input, FP32 or FP16 output of the same shape. axes: 0 = height, 1 = width, 2 = channel - what a computed
 * statistic is taken over; num_mean / num_std = 0 asks for that statistic to be computed per sample, else one value or
 * one per channel. */
RB200_API rb200_tensor rb200_normalize(rb200_context ctx, rb200_tensor in, const unsigned* axes, unsigned num_axes,
                                       const float* mean, unsigned num_mean, const float* std_dev, unsigned num_std,
                                       int is_output, float scale, float shift, int out_dtype);
/* rocalTranspose (rocal_api_augmentation.h:1338): perm over (height, width, channel); uint8 output whose dims are
 * {batch, d[perm[0]], d[perm[1]], d[perm[2]]} of the input's maximum shape, every sample at the origin of its slot. */
RB200_API rb200_tensor rb200_transpose(rb200_context ctx, rb200_tensor in, const unsigned* perm, unsigned num_perm,
                                       int is_output, int out_layout);
RB200_API rb200_tensor rb200_hue(rb200_context ctx, rb200_tensor in, int is_output, rb200_param hue, int out_layout,
                                 int out_dtype);
RB200_API rb200_tensor rb200_saturation(rb200_context ctx, rb200_tensor in, int is_output, rb200_param sat,
                                        int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_color_twist(rb200_context ctx, rb200_tensor in, int is_output, rb200_param alpha,
                                         rb200_param beta, rb200_param hue, rb200_param sat, int out_layout,
                                         int out_dtype);
RB200_API rb200_tensor rb200_warp_affine(rb200_context ctx, rb200_tensor in, int is_output, unsigned dest_height,
                                         unsigned dest_width, rb200_param x0, rb200_param x1, rb200_param y0,
                                         rb200_param y1, rb200_param o0, rb200_param o1, int interpolation,
                                         int out_layout, int out_dtype);
RB200_API rb200_tensor rb200_rotate(rb200_context ctx, rb200_tensor in, int is_output, rb200_param angle,
                                    unsigned dest_width, unsigned dest_height, int interpolation, int out_layout,
                                    int out_dtype);

/* ---- outputs: rocalGetOutputTensors (rocal_api_data_transfer.h:83) + rocalTensor accessors
 * (rocal_api_tensor.h:38-61). Output buffers are device memory owned by the context and stay valid
 * until the next rb200_run. ---- */
/* rocalSetOutputs (rocal_api_data_transfer.h:75): marks tensors as pipeline outputs; before rb200_verify. */
RB200_API int rb200_set_outputs(rb200_context ctx, const rb200_tensor* tensors, size_t n);
RB200_API size_t rb200_output_count(rb200_context ctx);
RB200_API rb200_tensor rb200_output(rb200_context ctx, size_t index);
RB200_API void* rb200_tensor_buffer(rb200_tensor t);
RB200_API unsigned rb200_tensor_num_dims(rb200_tensor t);
RB200_API void rb200_tensor_dims(rb200_tensor t, size_t* out_dims);
RB200_API void rb200_tensor_strides(rb200_tensor t, size_t* out_strides_bytes);
RB200_API int rb200_tensor_layout(rb200_tensor t);
RB200_API int rb200_tensor_dtype(rb200_tensor t);
RB200_API size_t rb200_tensor_data_size(rb200_tensor t);
/* rocalTensor::copy_data(user_buffer, mem_type): mem_type = RocalOutputMemType (0 host, 1 gpu, 2 pinned) */
RB200_API unsigned rb200_tensor_copy_data(rb200_tensor t, void* user_buffer, int mem_type);
/* rocalTensor::copy_roi: n x 4 unsigned (x, y, w, h) */
RB200_API void rb200_tensor_copy_roi(rb200_tensor t, void* roi_buffer);
/* DLPack export (__dlpack__ of rocAL_pybind/rocal_pybind.cpp:305-366, device type kDLCUDA): returns a
 * DLManagedTensor* whose deleter frees only the descriptor; the memory stays owned by the context. */
RB200_API void* rb200_tensor_dlpack(rb200_tensor t);
RB200_API int rb200_device_id(rb200_context ctx);
/* CUDA stream (cudaStream_t) the context launches on; outputs returned by rb200_run are complete. */
RB200_API void* rb200_stream(rb200_context ctx);
/* rocalToTensor (rocal_api_data_transfer.h:62-66): first output, uint8 -> fp32/fp16, x*multiplier+offset */
RB200_API int rb200_to_tensor(rb200_context ctx, void* out_ptr, int layout, int dtype, const float* multiplier3,
                              const float* offset3, int reverse_channels, int output_mem_type);

/* ---- SSD box encoder: rocalBoxEncoder / rocalCopyEncodedBoxesAndLables / rocalGetEncodedBoxesAndLables
 * (rocal_api_meta_data.h:270-286) ---- */
RB200_API int rb200_box_encoder(rb200_context ctx, const float* anchors_ltrb, size_t num_anchors, float criteria,
                                const float* means4, const float* stds4, int offset, float scale);
RB200_API int rb200_copy_encoded_boxes_and_labels(rb200_context ctx, float* boxes_buf, int* labels_buf);
RB200_API int rb200_get_encoded_boxes_and_labels(rb200_context ctx, float** boxes_dev, int** labels_dev,
                                                 size_t* num_anchors);

/* ---- box IoU matcher: rocalBoxIouMatcher / rocalGetMatchedIndices (rocal_api_meta_data.h:302-318).
 * Matched box index per anchor of the batch returned by the last rb200_run ([batch][num_anchors] int32 on
 * the device, valid until the next rb200_run); rb200_copy_matched_indices copies them to host memory. ---- */
RB200_API int rb200_box_iou_matcher(rb200_context ctx, const float* anchors_ltrb, size_t num_anchors, float high_threshold,
                                    float low_threshold, int allow_low_quality_matches);
RB200_API int rb200_get_matched_indices(rb200_context ctx, int** matches_dev, size_t* num_anchors);
RB200_API int rb200_copy_matched_indices(rb200_context ctx, int* matches_buf);

/* Boxes of the batch returned by the last rb200_run, after the graph's crops and mirrors: the data
 * of rocalGetBoundingBoxCount / rocalGetBoundingBoxCords / rocalGetBoundingBoxLabel
 * (rocal_api_meta_data.h:179-211) as flat arrays. Returns the total number of boxes; the arrays may be
 * NULL to query the size. counts holds one entry per sample. */
RB200_API size_t rb200_get_bounding_boxes(rb200_context ctx, float* ltrb, int* labels, int* counts);

/* [extension] Inspection of what the last returned batch used. rb200_get_crop_windows: n x {x, y, w, h}
 * source window of the crop-type operator (Crop*, CropMirrorNormalize, ResizeCropMirror, SSDRandomCrop)
 * that produced `t`. rb200_get_int_array / rb200_get_float_array: the current per-sample values of a
 * parameter (n = batch size; the parameter must be in use by a verified graph); they return the number
 * of values written. Parameters are process-wide objects that the loader thread renews for every batch it prepares:
 * with an external source fed one batch at a time the values are those of the batch rb200_run just returned; with a
 * folder or COCO source, which keeps the ring filled ahead, they already belong to the newest prepared batch. The
 * windows (rb200_get_crop_windows, rb200_get_decoder_crop_windows, rb200_get_bbox_crop_windows) and the boxes are kept
 * per batch and always describe the returned one. */
RB200_API int rb200_get_crop_windows(rb200_context ctx, rb200_tensor t, unsigned* xywh);
RB200_API size_t rb200_get_int_array(rb200_param p, int* out, size_t n);
RB200_API size_t rb200_get_float_array(rb200_param p, float* out, size_t n);
/* [extension] The same for the batch rb200_run returned, whatever the loader has prepared since: every batch keeps a
 * copy of the per-sample values it was built with. */
RB200_API size_t rb200_get_batch_int_array(rb200_context ctx, rb200_param p, int* out, size_t n);
RB200_API size_t rb200_get_batch_float_array(rb200_context ctx, rb200_param p, float* out, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* RB200_H */
