/*
 * tetris_b200.h -- C ABI of the B200 (sm_100a) sparse-filter convolution engine.
 *
 * Plain C: pointers, sizes and ints only.  Every entry point returns a status
 * code (TETRIS_OK == 0) instead of printing and calling exit() as the
 * reference's checkCudaErrors does (Tetris/cuda_utils.h:9-16); the text of the
 * last failure on the calling thread is available from tetris_last_error().
 *
 * What each entry point replaces in the reference (paths inside that project):
 *   tetris_filter_create*     SparseFilter<float,int,int> constructor: compress +
 *                             reorder + upload, Tetris/spconv2d_utils.h:25-265
 *   tetris_filter_destroy     ~SparseFilter, Tetris/spconv2d_utils.h:267-273
 *   tetris_filter_info/
 *   tetris_filter_download/
 *   tetris_filter_download_lists  the public fields and Get*() getters,
 *                             Tetris/spconv2d_utils.h:495-514
 *   tetris_conv2d_launch      SparseConv2d<...>() launcher,
 *                             Tetris/spconv2d_kernel.cu:163-188
 *   tetris_conv2d_time        TimingTetrisSparseConv2d, Tetris/spconv2d.cc:29-69
 *   tetris_conv2d_tune        GetTetrisSparseConv2dTime's tile search, Tetris/spconv2d.cc:72-329
 *   tetris_conv2d_host        CudaSparseConv2d's data path (host NCHW in, host
 *                             NCHW out), Tetris/spconv2d.cc:332-367
 *   tetris_conv2d_host_async/
 *   tetris_host_sync          no counterpart: the same data path, pipelined over slots
 *   tetris_nchw_to_nhwc/
 *   tetris_nhwc_to_nchw       NCHW2NHWC / NHWC2NCHW, Tetris/tensor_utils.cc:85-111,
 *                             done on the device
 *   tetris_filter_save/_load  no counterpart as calls: they replace REPEATING the constructor's
 *                             compress + upload (Tetris/spconv2d_utils.h:248-264) per process
 *                             and per timed tile configuration (Tetris/spconv2d.cc:285-311)
 *   tetris_conv2d_host_sharded  no counterpart (the reference pins device 0,
 *                             Tetris/spconv2d.cc:379-380): batch slices of one
 *                             call run on several GPUs of one box
 */
#ifndef TETRIS_B200_H_
#define TETRIS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TETRIS_OK = 0,
  TETRIS_ERR_INVALID = 1,     /* bad argument (null pointer, bad shape, ...)       */
  TETRIS_ERR_CUDA = 2,        /* a CUDA runtime call failed; see tetris_last_error */
  TETRIS_ERR_UNSUPPORTED = 3, /* shape outside what the kernels cover              */
  TETRIS_ERR_NOMEM = 4        /* host or device allocation failed                  */
};

/* Kernel variants accepted by tetris_conv2d_launch_ex. */
enum {
  TETRIS_VARIANT_AUTO = 0,    /* fastest kernel that covers the shape: the tuned choice if
                                 tetris_conv2d_tune ran for it, else the cost models'      */
  TETRIS_VARIANT_GENERIC = 1, /* one thread per output pixel, any KS/stride        */
  TETRIS_VARIANT_TILED = 2,   /* shared-memory tile, per-channel weight lists          */
                              /* 3 is retired (a jump-table interpreter kernel that measured
                                 slower than the list kernel); it is refused as invalid      */
  TETRIS_VARIANT_TENSOR = 4,  /* dense contraction on the tensor cores (tcgen05, split TF32);
                                 strides 1-8; in_channel <= 4, or a multiple of 4 with a
                                 16-byte aligned input                                    */
  TETRIS_VARIANT_TENSOR16 = 5 /* the same contraction in split FP16 (two 11-bit halves per
                                 operand, FP32 accumulate: FP32-accurate at twice the tensor
                                 rate); stride 1, in_channel a multiple of 4 and >= 8, 16-byte
                                 aligned input.  A launch whose largest |activation| is 2048
                                 or more (NaN, infinity) or below 2^-8 is recomputed on the
                                 device by the split-TF32 variant queued behind it         */
};

typedef struct tetris_filter tetris_filter_t; /* opaque; owns device buffers */

/* Compression options; zero in a field means "engine default". */
typedef struct {
  int oc_block;  /* output channels per register block, 8 (default) or 16            */
  int tile_ic;   /* input channels per stage, multiple of 4, <= 64                 */
  int deterministic; /* 1: bit-reproducible results from launch to launch (see tetris_conv2d_launch) */
  int reserved[5];
} tetris_filter_opts_t;

typedef struct {
  int in_channel, out_channel, kernel_size, groups;
  int oc_block, tile_ic;
  int n_oc_blocks;        /* ceil(out_channel / oc_block)                          */
  int n_stages;           /* ceil(in_channel / tile_ic)                            */
  int64_t nnz;            /* nonzero weights, padding excluded                     */
  int64_t n_ops;          /* 8-byte records in the compressed program stream       */
  int64_t compressed_bytes; /* device bytes held by both compressed forms          */
  int64_t n_list_units;   /* 8-byte units in the list form                         */
  int device;
  int reserved[5];
} tetris_filter_info_t;

/*
 * Compress a dense OIHW FP32 filter (host pointer, borrowed, read-only) on
 * `device` and keep the result there.  groups == 1, or groups == in_channel ==
 * out_channel (depthwise; filter is [C][1][KS][KS]).  The dense filter is
 * copied to the device and compressed there by CUDA kernels; nothing is
 * compressed on the host.
 */
int tetris_filter_create(const float *filter_oihw, int in_channel, int out_channel,
                         int kernel_size, int groups, int device, tetris_filter_t **out);
int tetris_filter_create_ex(const float *filter_oihw, int in_channel, int out_channel,
                            int kernel_size, int groups, int device,
                            const tetris_filter_opts_t *opts, tetris_filter_t **out);
void tetris_filter_destroy(tetris_filter_t *f);
int tetris_filter_info(const tetris_filter_t *f, tetris_filter_info_t *info);

/*
 * Copy the compressed program form back to the host: `ops` receives n_ops 8-byte
 * records, `prog_offsets` receives n_oc_blocks * n_stages + 1 record indices.
 * Either pointer may be NULL to skip that array.
 */
int tetris_filter_download(const tetris_filter_t *f, uint64_t *ops, size_t ops_capacity,
                           int32_t *prog_offsets, size_t offsets_capacity);

/* The same for the list form: n_list_units 8-byte units and the per-piece unit offsets. */
int tetris_filter_download_lists(const tetris_filter_t *f, uint64_t *units, size_t units_capacity,
                                 int32_t *list_offsets, size_t offsets_capacity);

/*
 * Waits for the device and reports whether any tensor-core launch of this filter gave up on one
 * of its bounded barrier waits since the last check (TETRIS_ERR_CUDA; the output of that launch
 * is invalid).  The other kernels have no waits that can fail.
 */
int tetris_filter_check(const tetris_filter_t *f);

/*
 * Convolution, device pointers, NHWC in and NHWC out as in the reference
 * launcher; asynchronous on `stream` (a cudaStream_t, may be NULL); allocates
 * nothing; the output is fully overwritten.  The device of `f` must be current.
 * Pointers need 4-byte alignment only; 16-byte aligned tensors take the vector paths (the
 * tensor-core variant needs a 16-byte aligned input and is not chosen without one).
 * Reproducibility: the list, generic and depthwise kernels add each output's taps in a fixed
 * order.  The tensor-core variant, on layers whose tiles fill the last wave of SMs badly, cuts
 * every tile's K range into 2-8 work items that ADD their partial results into the zeroed output
 * with floating-point atomics, in whatever order they finish: such a launch is not bit-identical
 * from run to run (differences of a few 1e-7 relative).  A filter created with
 * tetris_filter_opts_t.deterministic = 1 never splits and is bit-reproducible, at the cost of
 * the badly filled wave.
 */
int tetris_conv2d_launch(const tetris_filter_t *f, const float *d_input_nhwc,
                         float *d_output_nhwc, int batch_size, int img_h, int img_w,
                         int stride, int padding, void *stream);
int tetris_conv2d_launch_ex(const tetris_filter_t *f, const float *d_input_nhwc,
                            float *d_output_nhwc, int batch_size, int img_h, int img_w,
                            int stride, int padding, void *stream, int variant);

/*
 * The same launch with options fused into the kernel's store.  flags: TETRIS_FUSE_RELU -- the
 * output is max(y, 0).  The tensor-core variants rectify at their own store (and do not split a
 * tile's K range for such a launch); the other kernels are followed by an in-place pass on the
 * same stream.  No counterpart in the reference, whose kernel writes the plain convolution
 * (Tetris/spconv2d_kernel.cu:140-158).
 */
enum { TETRIS_FUSE_RELU = 1 };
int tetris_conv2d_launch_fused(const tetris_filter_t *f, const float *d_input_nhwc, float *d_output_nhwc,
                               int batch_size, int img_h, int img_w, int stride, int padding, void *stream,
                               int variant, int flags);

/*
 * Layer chains: the convolutions of a model run back to back on the device.  Layer i reads what
 * layer i - 1 left in HBM (NHWC), optionally rectified (relu) and 2x2 max-pooled (pool = 2; 0 =
 * none); the chain owns the activation buffers between the layers.  The reference has no chained
 * execution: it times isolated layers and adds the times up per model
 * (evalution/overall_speedup.py:159-165).
 *   tetris_chain_create   checks that the layers fit together (channels, extents) and allocates
 *                         the activations for `batch_size` images of img_h x img_w; all filters
 *                         must live on one device.  The filters stay the caller's.
 *   tetris_chain_run      queues every launch on `stream` (asynchronous, allocates nothing).
 *   tetris_chain_capture  runs the chain once, then captures it into a CUDA graph for this input
 *                         pointer; tetris_chain_replay launches that graph on `stream`.
 *   tetris_chain_output   the last layer's output (device pointer owned by the chain) and extent.
 *   tetris_chain_download waits for the device and copies that output (NHWC) to the host;
 *                         `capacity` in floats.
 */
typedef struct tetris_chain tetris_chain_t;
typedef struct {
  const tetris_filter_t *filter;
  int stride, padding;
  int relu;  /* 1: max(y, 0) after the convolution                       */
  int pool;  /* 2: 2x2 max-pooling, stride 2, after that; 0: none        */
} tetris_chain_layer_t;
int tetris_chain_create(const tetris_chain_layer_t *layers, int n_layers, int batch_size, int img_h, int img_w,
                        tetris_chain_t **out);
void tetris_chain_destroy(tetris_chain_t *c);
int tetris_chain_run(tetris_chain_t *c, const float *d_input_nhwc, void *stream);
int tetris_chain_capture(tetris_chain_t *c, const float *d_input_nhwc);
int tetris_chain_replay(tetris_chain_t *c, void *stream);
int tetris_chain_output(const tetris_chain_t *c, const float **d_output_nhwc, int *h, int *w, int *channels);
int tetris_chain_download(const tetris_chain_t *c, float *h_output_nhwc, size_t capacity);

/*
 * The reference's timing protocol: `warm` untimed launches, a device
 * synchronise, then `repeat` back-to-back launches between two events on
 * `stream`; *ms_mean = elapsed / repeat.
 */
int tetris_conv2d_time(const tetris_filter_t *f, const float *d_input_nhwc,
                       float *d_output_nhwc, int batch_size, int img_h, int img_w, int stride,
                       int padding, void *stream, int variant, int warm, int repeat,
                       float *ms_mean);

/*
 * Tile auto-tuning, the counterpart of the reference's search over its tile table
 * (GetTetrisSparseConv2dTime, Tetris/spconv2d.cc:72-329): times the `max_candidates` (0 = 12)
 * tile shapes / kernel instances that the engine's cost model ranks best, a few launches each,
 * remembers the fastest with the filter for this conv shape (later launches use it) and stores
 * its mean time in *best_ms (may be NULL).  Blocking; overwrites the output; untimed set-up work
 * in the reference's protocol.  The filter is not rebuilt: one compressed form serves every tile.
 */
int tetris_conv2d_tune(const tetris_filter_t *f, const float *d_input_nhwc, float *d_output_nhwc,
                       int batch_size, int img_h, int img_w, int stride, int padding, void *stream,
                       int max_candidates, float *best_ms);

/*
 * Which kernel a TETRIS_VARIANT_AUTO launch of this shape uses at the moment (the tuned choice if
 * tetris_conv2d_tune ran for the shape, else the cost models'): *variant receives
 * TETRIS_VARIANT_TILED, _TENSOR or _GENERIC (TETRIS_VARIANT_AUTO for a depthwise filter, which
 * has a single kernel).  No counterpart in the reference, which has one kernel.
 */
int tetris_conv2d_choice(const tetris_filter_t *f, int batch_size, int img_h, int img_w, int stride,
                         int padding, int *variant);

/*
 * Host NCHW in, host NCHW out, blocking.  Copies the input to the device,
 * transposes it to NHWC there, runs the convolution, transposes back and
 * copies the result out.  The device buffers come from a per-device workspace that
 * grows on demand and is kept between calls (tetris_release_workspace frees it).
 * `h_input` is not modified.
 */
int tetris_conv2d_host(const tetris_filter_t *f, const float *h_input_nchw,
                       float *h_output_nchw, int batch_size, int img_h, int img_w, int stride,
                       int padding, void *stream);

/*
 * The same data path without the final wait: the copies, transposes and the convolution are
 * queued on an internal stream selected by `slot` (0..3; each slot has its own stream and
 * workspace on the filter's device) and the call returns.  tetris_host_sync(device, slot) waits
 * for a slot (slot < 0: all of them); until then neither host buffer may be touched.  Calls that
 * alternate between slots overlap the upload of one with the download of the other.  Host buffers
 * should be page-locked for the copies to be asynchronous.  No counterpart in the reference,
 * whose CudaSparseConv2d is blocking.
 */
int tetris_conv2d_host_async(const tetris_filter_t *f, const float *h_input_nchw,
                             float *h_output_nchw, int batch_size, int img_h, int img_w, int stride,
                             int padding, int slot);
int tetris_host_sync(int device, int slot);

/* Frees the activation workspaces tetris_conv2d_host / _async keep on the devices it was used on. */
void tetris_release_workspace(void);

/* Device-side layout transposes (out of place), asynchronous on `stream`. */
int tetris_nchw_to_nhwc(const float *d_src, float *d_dst, int N, int C, int H, int W,
                        void *stream);
int tetris_nhwc_to_nchw(const float *d_src, float *d_dst, int N, int C, int H, int W,
                        void *stream);

/*
 * Batch partitioner: `filters[g]` is the same filter compressed on GPU g
 * (g < n_gpus).  The batch is cut into contiguous slices, slice g runs on the
 * device of filters[g] through tetris_conv2d_host from its own host thread; no
 * collective is involved.  Returns the first failing shard's status.
 */
int tetris_conv2d_host_sharded(tetris_filter_t *const *filters, int n_gpus,
                               const float *h_input_nchw, float *h_output_nchw,
                               int batch_size, int img_h, int img_w, int stride, int padding);

/* Contiguous batch slice [*begin, *begin + *count) of shard `rank` out of `world`. */
int tetris_batch_slice(int batch_size, int world, int rank, int *begin, int *count);

/* SM count, SM clock (kHz) and FP32 FMA lanes per SM of `device`. */
int tetris_device_info(int device, int *sm_count, int *sm_clock_khz, int *fp32_lanes_per_sm);

/*
 * No counterpart in the reference.  The piece offsets of the list form of a dense OIHW filter
 * that is ALREADY on the current device, written to `d_list_offsets`
 * (ceil(OC/oc_block) * ceil(IC/tile_ic) + 1 ints, device memory of the caller), asynchronous on
 * `stream` -- with no allocation of any kind, for callers that must not allocate where they
 * call: processes that gave all device memory to one pool at start-up and forbid cudaMalloc on
 * the request path, or code running inside another component's stream-ordered pipeline.  The
 * result equals the offsets tetris_filter_download_lists returns for the same filter and options
 * (the size a caller needs to reserve for the compressed filter is its last element + 2 units).
 *  - The per-piece counts live in a fixed 64 KiB array inside the library image (16384 pieces);
 *    more pieces than that are refused with TETRIS_ERR_UNSUPPORTED and a message.  Every GPU that
 *    loads the library holds that array until the process exits.
 *  - The first call on a device looks up the array's device address (once per device, that
 *    device being current) and, where the CUDA runtime loads code lazily, may load the library's
 *    kernels; make that first call at start-up, before any stream capture begins.
 *  - Both pointers are checked to be device memory of the current device (TETRIS_ERR_INVALID
 *    otherwise); the check is a query and allocates nothing.
 *  - All calls share the array, so two calls that can overlap on the GPU (different streams, or
 *    different host threads) race on it; keep calls on one device in stream order.  Nothing has
 *    to be cleared between calls: each call rewrites every count it later reads.
 */
int tetris_list_offsets_noalloc(const float *d_filter_oihw, int in_channel, int out_channel,
                                int kernel_size, int oc_block, int tile_ic,
                                int32_t *d_list_offsets, void *stream);

/*
 * Compressed-filter files.  The reference recompresses every filter in every process and once
 * per tile configuration it times (upload at Tetris/spconv2d_utils.h:248-264, rebuild loop at
 * Tetris/spconv2d.cc:285-311); these three calls make that a one-off.
 *   tetris_filter_save        writes both compressed forms as they lie on the device (for a
 *                             depthwise filter its dense taps) and the tile plans
 *                             tetris_conv2d_tune has chosen so far, behind a versioned header
 *                             with a checksum.
 *   tetris_filter_load        reads such a file onto `device`: same downloads, same launches and
 *                             the same tuned choices as the filter that was saved.  The
 *                             tensor-core tile images are rebuilt on the device from the list form.
 *   tetris_filter_file_check  validates a file on the host alone (no GPU): header, sizes,
 *                             offsets, checksum; fills `info` (may be NULL; info->device = -1).
 * A missing, truncated, foreign or damaged file is TETRIS_ERR_INVALID with the reason in
 * tetris_last_error().
 */
int tetris_filter_save(const tetris_filter_t *f, const char *path);
int tetris_filter_load(const char *path, int device, tetris_filter_t **out);
int tetris_filter_file_check(const char *path, tetris_filter_info_t *info);

/*
 * Number of convolution kernels the library has launched in this process so far (every variant,
 * every device and thread; tuning launches included).  No counterpart in the reference; lets a
 * harness check that a timing loop really issued warm + repeat launches.
 */
unsigned long long tetris_launch_count(void);

/*
 * Failure-detection test hook (no counterpart in the reference, whose kernels have no waits that
 * can fail).  Every barrier wait inside the tensor-core kernels is bounded; when one runs out the
 * kernel raises a flag, lets every role drain (loads, copies and MMAs already started are waited
 * for), frees its tensor memory and returns, and tetris_filter_check reports TETRIS_ERR_CUDA once.
 * tetris_test_inject(TETRIS_INJECT_WITHHOLD_LOAD, n) makes the following tensor-core launches of
 * this process leave out every CTA's first activation load and give up after n polls (0: the
 * built-in limit, seconds), so that a test can see that path end to end without a GPU fault: the
 * launch returns normally, its output is unspecified, the context stays usable.
 * tetris_test_inject(TETRIS_INJECT_NONE, 0) switches it off.  Never use it outside tests.
 */
#define TETRIS_INJECT_NONE 0
#define TETRIS_INJECT_WITHHOLD_LOAD 1
int tetris_test_inject(int what, unsigned spin_limit);

/* Text of the last error raised on this thread ("" if none). */
const char *tetris_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* TETRIS_B200_H_ */
