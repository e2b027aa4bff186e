// The C ABI (include/tetris_b200.h): argument checks, handle lifetime, kernel selection, the
// reference's timing protocol, the host-pointer data path and the batch partitioner.
#include <stdarg.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "internal.h"

namespace tetris {

static thread_local char g_error[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
static std::atomic<int> g_inject{0};
static std::atomic<unsigned> g_inject_spin{0};
int test_injection(unsigned *spin_limit) {
  const int what = g_inject.load(std::memory_order_relaxed);
  *spin_limit = what ? g_inject_spin.load(std::memory_order_relaxed) : 0u;
  return what == TETRIS_INJECT_WITHHOLD_LOAD ? 1 : 0;
}

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {

// Activation workspace of tetris_conv2d_host, one per device, grown on demand.
struct Workspace {
  std::mutex mutex;
  void *ptr = nullptr;
  size_t bytes = 0;
};
constexpr int kMaxWsDevices = 64;
Workspace g_workspace[kMaxWsDevices];

// Makes `device` current for the lifetime of the object and restores the previous one.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    ok = cudaSetDevice(device) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

int make_shape(const tetris_filter *f, int batch, int h, int w, int stride, int padding,
               ConvShape *s) {
  if (!f) { set_error("filter handle is NULL"); return TETRIS_ERR_INVALID; }
  if (batch < 0 || h < 1 || w < 1 || stride < 1 || padding < 0) {
    set_error("bad conv shape: batch=%d h=%d w=%d stride=%d padding=%d", batch, h, w, stride, padding);
    return TETRIS_ERR_INVALID;
  }
  s->N = batch; s->H = h; s->W = w; s->IC = f->in_channel; s->OC = f->out_channel;
  s->KS = f->kernel_size; s->S = stride; s->P = padding;
  // output extent as in Tetris/spconv2d.cc:339-340
  s->OH = (h + 2 * padding - f->kernel_size) / stride + 1;
  s->OW = (w + 2 * padding - f->kernel_size) / stride + 1;
  if (h + 2 * padding < f->kernel_size || w + 2 * padding < f->kernel_size) {
    set_error("image %dx%d (+pad %d) smaller than the %dx%d kernel", h, w, padding,
              f->kernel_size, f->kernel_size);
    return TETRIS_ERR_INVALID;
  }
  return TETRIS_OK;
}

thread_local bool tl_relu_fused = false;

int dispatch_kernel(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                    cudaStream_t st, int variant);

// One convolution launch.  A requested ReLU is applied at the kernel's own store where the
// kernel can do that (the tensor-core variants), else by an in-place pass behind it.
int dispatch(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
             cudaStream_t st, int variant) {
  tl_relu_fused = false;
  const int rc = dispatch_kernel(f, in, out, s, st, variant);
  if (rc || !s.relu || tl_relu_fused || s.N == 0) return rc;
  return launch_relu_inplace(out, (size_t)s.N * s.OH * s.OW * s.OC, st);
}

int dispatch_kernel(const tetris_filter *f, const float *in, float *out, const ConvShape &s,
                    cudaStream_t st, int variant) {
  if (s.N == 0) return TETRIS_OK;
  if (f->groups != 1) return launch_depthwise(f, in, out, s, st);
  switch (variant) {
    case TETRIS_VARIANT_GENERIC: return launch_conv_generic(f, in, out, s, st);
    case TETRIS_VARIANT_TILED: return launch_conv_tiled(f, in, out, s, st, false);
    case TETRIS_VARIANT_TENSOR: return launch_conv_tc(f, in, out, s, st);
    case TETRIS_VARIANT_TENSOR16: return launch_conv_tc16(f, in, out, s, st);
    case TETRIS_VARIANT_AUTO: {
      // the list kernel (which may hand over to the tensor-core variant); when no tile geometry of
      // it fits shared memory (long list pieces of a dense, large filter with a caller-chosen
      // stage size) the tensor-core variant if it covers the shape, else the generic kernel
      if (conv_tiled_supported(f, s)) {
        const int rc = launch_conv_tiled(f, in, out, s, st, true);
        if (rc != TETRIS_ERR_UNSUPPORTED) return rc;
      }
      if (conv_tc_supported(f, s) && (reinterpret_cast<uintptr_t>(in) & 15) == 0)
        return launch_conv_tc(f, in, out, s, st);
      return launch_conv_generic(f, in, out, s, st);
    }
    default: set_error("unknown kernel variant %d", variant); return TETRIS_ERR_INVALID;
  }
}

}  // namespace

void note_relu_fused() { tl_relu_fused = true; }

int conv_dispatch_auto(const tetris_filter *f, const float *in, float *out, const ConvShape &s, cudaStream_t st) {
  return dispatch(f, in, out, s, st, TETRIS_VARIANT_AUTO);
}

}  // namespace tetris

using namespace tetris;

extern "C" {

const char *tetris_last_error(void) { return g_error; }

unsigned long long tetris_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int tetris_test_inject(int what, unsigned spin_limit) {
  if (what != TETRIS_INJECT_NONE && what != TETRIS_INJECT_WITHHOLD_LOAD) {
    tetris::set_error("tetris_test_inject: unknown injection %d", what);
    return TETRIS_ERR_INVALID;
  }
  tetris::g_inject_spin.store(spin_limit, std::memory_order_relaxed);
  tetris::g_inject.store(what, std::memory_order_relaxed);
  return TETRIS_OK;
}

int tetris_filter_create(const float *filter_oihw, int in_channel, int out_channel,
                         int kernel_size, int groups, int device, tetris_filter_t **out) {
  return tetris_filter_create_ex(filter_oihw, in_channel, out_channel, kernel_size, groups, device,
                                 nullptr, out);
}

int tetris_filter_create_ex(const float *filter_oihw, int in_channel, int out_channel,
                            int kernel_size, int groups, int device,
                            const tetris_filter_opts_t *opts, tetris_filter_t **out) {
  if (!filter_oihw || !out) { set_error("filter or out pointer is NULL"); return TETRIS_ERR_INVALID; }
  *out = nullptr;
  if (in_channel < 1 || out_channel < 1 || kernel_size < 1 || kernel_size > 8) {
    set_error("bad filter shape: ic=%d oc=%d ks=%d (ks must be 1..8)", in_channel, out_channel,
              kernel_size);
    return TETRIS_ERR_INVALID;
  }
  const bool depthwise = groups != 1;
  if (depthwise && !(groups == in_channel && groups == out_channel)) {
    set_error("groups=%d: only 1 or depthwise (groups == ic == oc) is supported", groups);
    return TETRIS_ERR_UNSUPPORTED;
  }
  const int K = opts && opts->oc_block ? opts->oc_block : 8;
  const bool auto_tic = !(opts && opts->tile_ic);
  // engine default: up to about 144 filter taps per channel block and stage (16 channels for 3x3,
  // 32 for 1x1), halved below while the longest list piece is too long for shared memory
  int TIC = auto_tic ? (kernel_size == 1 ? 32 : kernel_size == 2 ? 32 : kernel_size <= 4 ? 16 : 8)
                     : opts->tile_ic;
  if (!(K == 8 || K == 16) || TIC < 4 || TIC > kMaxTileIc || (TIC & 3)) {
    set_error("bad compression options: oc_block=%d tile_ic=%d", K, TIC);
    return TETRIS_ERR_INVALID;
  }
  int n_dev = 0;
  TETRIS_CUDA_TRY(cudaGetDeviceCount(&n_dev));
  if (device < 0 || device >= n_dev) {
    set_error("device %d out of range (%d visible)", device, n_dev);
    return TETRIS_ERR_INVALID;
  }
  DeviceGuard guard(device);
  if (!guard.ok) { set_error("cudaSetDevice(%d) failed", device); return TETRIS_ERR_CUDA; }

  tetris_filter *f = new (std::nothrow) tetris_filter();
  if (!f) { set_error("out of host memory"); return TETRIS_ERR_NOMEM; }
  memset(f, 0, sizeof(*f));
  f->in_channel = in_channel; f->out_channel = out_channel; f->kernel_size = kernel_size;
  f->groups = groups; f->device = device;
  f->oc_block = K; f->tile_ic = TIC;
  f->deterministic = opts && opts->deterministic ? 1 : 0;
  f->plan_cache = tiled_plan_cache_new();

  const size_t per_oc = depthwise ? 1 : (size_t)in_channel;
  const size_t dense_bytes = (size_t)out_channel * per_oc * kernel_size * kernel_size * sizeof(float);
  float *d_dense = nullptr;
  int32_t *d_scratch = nullptr;
  int rc = TETRIS_OK;
  auto fail = [&](int code) {
    cudaFree(d_dense); cudaFree(d_scratch);
    f->d_dense = nullptr;
    tetris_filter_destroy(f);
    return code;
  };
  if (cudaMalloc(&d_dense, dense_bytes) != cudaSuccess) {
    cudaGetLastError();
    set_error("cudaMalloc of %zu bytes for the dense filter failed", dense_bytes);
    return fail(TETRIS_ERR_NOMEM);
  }
  if (cudaMemcpy(d_dense, filter_oihw, dense_bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
    set_error("copy of the dense filter to the device failed");
    return fail(TETRIS_ERR_CUDA);
  }
  if (depthwise) {
    // Dense on purpose: kept as is, counted for the info block.
    f->d_dense = d_dense;
    f->n_oc_blocks = 0; f->n_stages = 0; f->n_ops = 0;
    int64_t nnz = 0;
    for (size_t i = 0; i < dense_bytes / sizeof(float); ++i) nnz += filter_oihw[i] != 0.f;
    f->nnz = nnz;
    *out = f;
    return TETRIS_OK;
  }

  // List pieces are staged in shared memory by the tiled kernel, so their length is bounded:
  // when the stage size is left to the engine, halve it until the longest piece is short enough.
  constexpr int kPieceUnitsTarget = 640;
  const int B = (out_channel + K - 1) / K;
  int T = 0, P = 0;
  std::vector<int32_t> h_offsets;
  auto alloc_offsets = [&](int32_t **d_offsets) {
    cudaFree(d_scratch); cudaFree(*d_offsets);
    d_scratch = nullptr; *d_offsets = nullptr;
    return cudaMalloc(&d_scratch, compress_scratch_bytes(P)) == cudaSuccess &&
           cudaMalloc(d_offsets, (size_t)(P + 1) * sizeof(int32_t)) == cudaSuccess;
  };
  auto fetch_offsets = [&](const int32_t *d_offsets, int *longest) {
    h_offsets.resize(P + 1);
    if (cudaMemcpy(h_offsets.data(), d_offsets, (size_t)(P + 1) * sizeof(int32_t),
                   cudaMemcpyDeviceToHost) != cudaSuccess)
      return false;
    *longest = 0;
    for (int i = 0; i < P; ++i) *longest = std::max(*longest, h_offsets[i + 1] - h_offsets[i]);
    return true;
  };
  // ---- LIST form (tiled kernel) ----
  for (;;) {
    T = (in_channel + TIC - 1) / TIC;
    P = B * T;
    if (!alloc_offsets(&f->d_list_offsets)) {
      cudaGetLastError();
      set_error("cudaMalloc of compressor scratch failed");
      return fail(TETRIS_ERR_NOMEM);
    }
    if ((rc = list_count(d_dense, in_channel, out_channel, kernel_size, K, TIC, B, T, d_scratch, 0)) ||
        (rc = compress_scan(d_scratch, f->d_list_offsets, P, 0)))
      return fail(rc);
    if (!fetch_offsets(f->d_list_offsets, &f->max_list_units)) {
      set_error("compressor count/scan failed: %s", cudaGetErrorString(cudaGetLastError()));
      return fail(TETRIS_ERR_CUDA);
    }
    if (!auto_tic || f->max_list_units <= kPieceUnitsTarget || TIC <= 4) break;
    TIC /= 2;
  }
  f->tile_ic = TIC;
  f->n_oc_blocks = B; f->n_stages = T;
  f->n_list_units = (int64_t)h_offsets[P] + 2;
  if (cudaMalloc(&f->d_lists, (size_t)f->n_list_units * sizeof(uint64_t)) != cudaSuccess) {
    cudaGetLastError();
    set_error("cudaMalloc of %lld list units failed", (long long)f->n_list_units);
    return fail(TETRIS_ERR_NOMEM);
  }
  if ((rc = list_fill(d_dense, in_channel, out_channel, kernel_size, K, TIC, B, T,
                      f->d_list_offsets, f->d_lists, f->n_list_units, 0)))
    return fail(rc);
  // ---- PROGRAM form (generic kernel) ----
  if (!alloc_offsets(&f->d_prog_offsets)) {
    cudaGetLastError();
    set_error("cudaMalloc of compressor scratch failed");
    return fail(TETRIS_ERR_NOMEM);
  }
  if ((rc = compress_count(d_dense, in_channel, out_channel, kernel_size, K, TIC, B, T, d_scratch, 0)) ||
      (rc = compress_scan(d_scratch, f->d_prog_offsets, P, 0)))
    return fail(rc);
  unsigned long long nnz = 0;
  if (!fetch_offsets(f->d_prog_offsets, &f->max_prog_ops) ||
      cudaMemcpy(&nnz, compress_nnz_ptr(d_scratch, P), sizeof(nnz), cudaMemcpyDeviceToHost) != cudaSuccess) {
    set_error("compressor count/scan failed: %s", cudaGetErrorString(cudaGetLastError()));
    return fail(TETRIS_ERR_CUDA);
  }
  const int32_t total = h_offsets[P];
  f->nnz = (int64_t)nnz;
  f->n_ops = (int64_t)total + kTailPadOps;
  if (cudaMalloc(&f->d_ops, (size_t)f->n_ops * sizeof(uint64_t)) != cudaSuccess) {
    cudaGetLastError();
    set_error("cudaMalloc of %lld program records failed", (long long)f->n_ops);
    return fail(TETRIS_ERR_NOMEM);
  }
  if ((rc = compress_fill(d_dense, in_channel, out_channel, kernel_size, K, TIC, B, T,
                          f->d_prog_offsets, f->d_ops, f->n_ops, 0)))
    return fail(rc);
  if ((rc = conv_tc_prepare(f, d_dense)) || (rc = conv_tc16_prepare(f, d_dense))) return fail(rc);
  if (cudaDeviceSynchronize() != cudaSuccess) {
    set_error("compressor fill failed: %s", cudaGetErrorString(cudaGetLastError()));
    return fail(TETRIS_ERR_CUDA);
  }
  cudaFree(d_dense);
  cudaFree(d_scratch);
  *out = f;
  return TETRIS_OK;
}

void tetris_filter_destroy(tetris_filter_t *f) {
  if (!f) return;
  DeviceGuard guard(f->device);
  cudaFree(f->d_ops);
  cudaFree(f->d_prog_offsets);
  cudaFree(f->d_lists);
  cudaFree(f->d_list_offsets);
  tiled_plan_cache_delete(f->plan_cache);
  conv_tc_state_delete(f->tc_state);
  conv_tc16_state_delete(f->tc16_state);
  cudaFree(f->d_dense);
  delete f;
}

int tetris_filter_info(const tetris_filter_t *f, tetris_filter_info_t *info) {
  if (!f || !info) { set_error("NULL argument"); return TETRIS_ERR_INVALID; }
  memset(info, 0, sizeof(*info));
  info->in_channel = f->in_channel; info->out_channel = f->out_channel;
  info->kernel_size = f->kernel_size; info->groups = f->groups;
  info->oc_block = f->oc_block; info->tile_ic = f->tile_ic;
  info->n_oc_blocks = f->n_oc_blocks; info->n_stages = f->n_stages;
  info->nnz = f->nnz; info->n_ops = f->n_ops; info->n_list_units = f->n_list_units;
  info->compressed_bytes =
      f->groups != 1
          ? (int64_t)f->out_channel * f->kernel_size * f->kernel_size * (int64_t)sizeof(float)
          : (f->n_ops + f->n_list_units) * (int64_t)sizeof(uint64_t) +
                2 * ((int64_t)f->n_oc_blocks * f->n_stages + 1) * (int64_t)sizeof(int32_t);
  info->device = f->device;
  return TETRIS_OK;
}

int tetris_filter_download(const tetris_filter_t *f, uint64_t *ops, size_t ops_capacity,
                           int32_t *prog_offsets, size_t offsets_capacity) {
  if (!f) { set_error("filter handle is NULL"); return TETRIS_ERR_INVALID; }
  if (f->groups != 1) { set_error("a depthwise filter has no program stream"); return TETRIS_ERR_UNSUPPORTED; }
  DeviceGuard guard(f->device);
  if (ops) {
    if (ops_capacity < (size_t)f->n_ops) { set_error("ops buffer too small"); return TETRIS_ERR_INVALID; }
    TETRIS_CUDA_TRY(cudaMemcpy(ops, f->d_ops, (size_t)f->n_ops * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  }
  if (prog_offsets) {
    const size_t n = (size_t)f->n_oc_blocks * f->n_stages + 1;
    if (offsets_capacity < n) { set_error("offsets buffer too small"); return TETRIS_ERR_INVALID; }
    TETRIS_CUDA_TRY(cudaMemcpy(prog_offsets, f->d_prog_offsets, n * sizeof(int32_t), cudaMemcpyDeviceToHost));
  }
  return TETRIS_OK;
}

int tetris_filter_download_lists(const tetris_filter_t *f, uint64_t *units, size_t units_capacity,
                                 int32_t *list_offsets, size_t offsets_capacity) {
  if (!f) { set_error("filter handle is NULL"); return TETRIS_ERR_INVALID; }
  if (f->groups != 1) { set_error("a depthwise filter has no lists"); return TETRIS_ERR_UNSUPPORTED; }
  DeviceGuard guard(f->device);
  if (units) {
    if (units_capacity < (size_t)f->n_list_units) { set_error("units buffer too small"); return TETRIS_ERR_INVALID; }
    TETRIS_CUDA_TRY(cudaMemcpy(units, f->d_lists, (size_t)f->n_list_units * sizeof(uint64_t), cudaMemcpyDeviceToHost));
  }
  if (list_offsets) {
    const size_t n = (size_t)f->n_oc_blocks * f->n_stages + 1;
    if (offsets_capacity < n) { set_error("offsets buffer too small"); return TETRIS_ERR_INVALID; }
    TETRIS_CUDA_TRY(cudaMemcpy(list_offsets, f->d_list_offsets, n * sizeof(int32_t), cudaMemcpyDeviceToHost));
  }
  return TETRIS_OK;
}

int tetris_filter_check(const tetris_filter_t *f) {
  if (!f) { set_error("filter handle is NULL"); return TETRIS_ERR_INVALID; }
  DeviceGuard guard(f->device);
  if (cudaDeviceSynchronize() != cudaSuccess) {
    set_error("device error: %s", cudaGetErrorString(cudaGetLastError()));
    return TETRIS_ERR_CUDA;
  }
  if (f->groups != 1 && depthwise_check_error()) {
    set_error("a depthwise launch gave up on a bounded barrier wait; its output is invalid");
    return TETRIS_ERR_CUDA;
  }
  if (conv_tc_check_error(f) | conv_tc16_check_error(f)) {
    set_error("a tensor-core launch of this filter gave up on a bounded barrier wait; its output is invalid");
    return TETRIS_ERR_CUDA;
  }
  return TETRIS_OK;
}

int tetris_conv2d_launch_ex(const tetris_filter_t *f, const float *d_input_nhwc,
                            float *d_output_nhwc, int batch_size, int img_h, int img_w,
                            int stride, int padding, void *stream, int variant) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (batch_size > 0 && (!d_input_nhwc || !d_output_nhwc)) {
    set_error("input or output pointer is NULL");
    return TETRIS_ERR_INVALID;
  }
  return dispatch(f, d_input_nhwc, d_output_nhwc, s, (cudaStream_t)stream, variant);
}

int tetris_conv2d_launch_fused(const tetris_filter_t *f, const float *d_input_nhwc, float *d_output_nhwc,
                               int batch_size, int img_h, int img_w, int stride, int padding, void *stream,
                               int variant, int flags) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (batch_size > 0 && (!d_input_nhwc || !d_output_nhwc)) { set_error("input or output pointer is NULL"); return TETRIS_ERR_INVALID; }
  if (flags & ~TETRIS_FUSE_RELU) { set_error("unknown fusion flags 0x%x", flags); return TETRIS_ERR_INVALID; }
  s.relu = (flags & TETRIS_FUSE_RELU) ? 1 : 0;
  return dispatch(f, d_input_nhwc, d_output_nhwc, s, (cudaStream_t)stream, variant);
}

int tetris_conv2d_launch(const tetris_filter_t *f, const float *d_input_nhwc,
                         float *d_output_nhwc, int batch_size, int img_h, int img_w,
                         int stride, int padding, void *stream) {
  return tetris_conv2d_launch_ex(f, d_input_nhwc, d_output_nhwc, batch_size, img_h, img_w, stride,
                                 padding, stream, TETRIS_VARIANT_AUTO);
}

int tetris_conv2d_time(const tetris_filter_t *f, const float *d_input_nhwc,
                       float *d_output_nhwc, int batch_size, int img_h, int img_w, int stride,
                       int padding, void *stream, int variant, int warm, int repeat,
                       float *ms_mean) {
  if (!ms_mean || repeat < 1 || warm < 0) { set_error("bad timing arguments"); return TETRIS_ERR_INVALID; }
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (!d_input_nhwc || !d_output_nhwc) { set_error("input or output pointer is NULL"); return TETRIS_ERR_INVALID; }
  cudaStream_t st = (cudaStream_t)stream;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  TETRIS_CUDA_TRY(cudaEventCreate(&e0));
  if (cudaEventCreate(&e1) != cudaSuccess) { cudaEventDestroy(e0); set_error("cudaEventCreate failed"); return TETRIS_ERR_CUDA; }
  auto done = [&](int code) { cudaEventDestroy(e0); cudaEventDestroy(e1); return code; };
  for (int i = 0; i < warm; ++i)
    if ((rc = dispatch(f, d_input_nhwc, d_output_nhwc, s, st, variant))) return done(rc);
  if (cudaDeviceSynchronize() != cudaSuccess) {
    set_error("warm-up failed: %s", cudaGetErrorString(cudaGetLastError()));
    return done(TETRIS_ERR_CUDA);
  }
  cudaEventRecord(e0, st);
  for (int i = 0; i < repeat; ++i)
    if ((rc = dispatch(f, d_input_nhwc, d_output_nhwc, s, st, variant))) return done(rc);
  cudaEventRecord(e1, st);
  if (cudaEventSynchronize(e1) != cudaSuccess) {
    set_error("timed launches failed: %s", cudaGetErrorString(cudaGetLastError()));
    return done(TETRIS_ERR_CUDA);
  }
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  *ms_mean = ms / (float)repeat;
  return done(TETRIS_OK);
}

int tetris_conv2d_tune(const tetris_filter_t *f, const float *d_input_nhwc, float *d_output_nhwc,
                       int batch_size, int img_h, int img_w, int stride, int padding, void *stream,
                       int max_candidates, float *best_ms) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (!d_input_nhwc || !d_output_nhwc || batch_size < 1) { set_error("tuning needs real buffers and a non-empty batch"); return TETRIS_ERR_INVALID; }
  if (max_candidates < 1) max_candidates = 12;
  if (f->groups != 1 || !conv_tiled_supported(f, s)) {  // nothing to choose between: report the time
    float ms = 0.f;
    rc = tetris_conv2d_time(f, d_input_nhwc, d_output_nhwc, batch_size, img_h, img_w, stride, padding,
                            stream, TETRIS_VARIANT_AUTO, 2, 5, &ms);
    if (!rc && best_ms) *best_ms = ms;
    return rc;
  }
  return tune_conv_tiled(f, d_input_nhwc, d_output_nhwc, s, (cudaStream_t)stream, max_candidates, best_ms);
}

int tetris_conv2d_choice(const tetris_filter_t *f, int batch_size, int img_h, int img_w, int stride,
                         int padding, int *variant) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (!variant) { set_error("variant pointer is NULL"); return TETRIS_ERR_INVALID; }
  if (f->groups != 1) { *variant = TETRIS_VARIANT_AUTO; return TETRIS_OK; }  // depthwise: one kernel
  if (conv_tiled_supported(f, s)) {
    rc = conv_auto_choice(f, s, variant);
    if (rc != TETRIS_ERR_UNSUPPORTED) return rc;
  }
  *variant = conv_tc_supported(f, s) ? TETRIS_VARIANT_TENSOR : TETRIS_VARIANT_GENERIC;
  return TETRIS_OK;
}

int tetris_nchw_to_nhwc(const float *d_src, float *d_dst, int N, int C, int H, int W, void *stream) {
  if (!d_src || !d_dst || N < 0 || C < 1 || H < 1 || W < 1) { set_error("bad layout arguments"); return TETRIS_ERR_INVALID; }
  return launch_nchw_to_nhwc(d_src, d_dst, N, C, H, W, (cudaStream_t)stream);
}
int tetris_nhwc_to_nchw(const float *d_src, float *d_dst, int N, int C, int H, int W, void *stream) {
  if (!d_src || !d_dst || N < 0 || C < 1 || H < 1 || W < 1) { set_error("bad layout arguments"); return TETRIS_ERR_INVALID; }
  return launch_nhwc_to_nchw(d_src, d_dst, N, C, H, W, (cudaStream_t)stream);
}

int tetris_conv2d_host(const tetris_filter_t *f, const float *h_input_nchw,
                       float *h_output_nchw, int batch_size, int img_h, int img_w, int stride,
                       int padding, void *stream) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (batch_size == 0) return TETRIS_OK;
  if (!h_input_nchw || !h_output_nchw) { set_error("input or output pointer is NULL"); return TETRIS_ERR_INVALID; }
  DeviceGuard guard(f->device);
  if (!guard.ok) { set_error("cudaSetDevice(%d) failed", f->device); return TETRIS_ERR_CUDA; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t in_elems = (size_t)s.N * s.IC * s.H * s.W, out_elems = (size_t)s.N * s.OC * s.OH * s.OW;
  // One buffer: [input NCHW | input NHWC | output NHWC | output NCHW].  It comes from a
  // grow-only per-device workspace that is kept between calls (tetris_release_workspace frees
  // it); a call that finds the workspace in use by another thread allocates its own.
  const size_t need = (2 * in_elems + 2 * out_elems) * sizeof(float);
  Workspace *ws = f->device < kMaxWsDevices ? &g_workspace[f->device] : nullptr;
  const bool cached = ws && ws->mutex.try_lock();
  float *d = nullptr;
  if (cached) {
    if (ws->bytes < need) {
      cudaFree(ws->ptr);
      ws->ptr = nullptr; ws->bytes = 0;
      if (cudaMalloc(&ws->ptr, need) == cudaSuccess) ws->bytes = need;
    }
    d = static_cast<float *>(ws->ptr);
  } else if (cudaMalloc(&d, need) != cudaSuccess) {
    d = nullptr;
  }
  if (!d) {
    cudaGetLastError();
    if (cached) ws->mutex.unlock();
    set_error("cudaMalloc of %zu bytes of activations failed", need);
    return TETRIS_ERR_NOMEM;
  }
  float *d_in_nchw = d, *d_in_nhwc = d + in_elems, *d_out_nhwc = d + 2 * in_elems,
        *d_out_nchw = d + 2 * in_elems + out_elems;
  auto done = [&](int code) {
    if (cached) ws->mutex.unlock(); else cudaFree(d);
    return code;
  };
  if (cudaMemcpyAsync(d_in_nchw, h_input_nchw, in_elems * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess) {
    set_error("host-to-device copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    return done(TETRIS_ERR_CUDA);
  }
  if ((rc = launch_nchw_to_nhwc(d_in_nchw, d_in_nhwc, s.N, s.IC, s.H, s.W, st))) return done(rc);
  if ((rc = dispatch(f, d_in_nhwc, d_out_nhwc, s, st, TETRIS_VARIANT_AUTO))) return done(rc);
  if ((rc = launch_nhwc_to_nchw(d_out_nhwc, d_out_nchw, s.N, s.OC, s.OH, s.OW, st))) return done(rc);
  if (cudaMemcpyAsync(h_output_nchw, d_out_nchw, out_elems * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    set_error("convolution or device-to-host copy failed: %s", cudaGetErrorString(cudaGetLastError()));
    return done(TETRIS_ERR_CUDA);
  }
  return done(TETRIS_OK);
}

// ---- pipelined host-pointer path: `slot` selects one of kSlots (stream, workspace) pairs per
//      device, so the upload of one call overlaps the download of the previous one ----
namespace {
constexpr int kSlots = 4;
struct HostSlot {
  std::mutex mutex;
  cudaStream_t stream = nullptr;
  void *ptr = nullptr;
  size_t bytes = 0;
};
HostSlot g_slots[kMaxWsDevices][kSlots];
}  // namespace

int tetris_conv2d_host_async(const tetris_filter_t *f, const float *h_input_nchw,
                             float *h_output_nchw, int batch_size, int img_h, int img_w, int stride,
                             int padding, int slot) {
  ConvShape s;
  int rc = make_shape(f, batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (slot < 0 || slot >= kSlots || f->device >= kMaxWsDevices) {
    set_error("slot %d outside [0, %d)", slot, kSlots);
    return TETRIS_ERR_INVALID;
  }
  if (batch_size == 0) return TETRIS_OK;
  if (!h_input_nchw || !h_output_nchw) { set_error("input or output pointer is NULL"); return TETRIS_ERR_INVALID; }
  DeviceGuard guard(f->device);
  if (!guard.ok) { set_error("cudaSetDevice(%d) failed", f->device); return TETRIS_ERR_CUDA; }
  HostSlot &hs = g_slots[f->device][slot];
  std::lock_guard<std::mutex> lock(hs.mutex);
  if (!hs.stream) TETRIS_CUDA_TRY(cudaStreamCreateWithFlags(&hs.stream, cudaStreamNonBlocking));
  const size_t in_elems = (size_t)s.N * s.IC * s.H * s.W, out_elems = (size_t)s.N * s.OC * s.OH * s.OW;
  const size_t need = (2 * in_elems + 2 * out_elems) * sizeof(float);
  if (hs.bytes < need) {
    // the slot's earlier work may still read the old buffer
    TETRIS_CUDA_TRY(cudaStreamSynchronize(hs.stream));
    cudaFree(hs.ptr);
    hs.ptr = nullptr; hs.bytes = 0;
    if (cudaMalloc(&hs.ptr, need) != cudaSuccess) {
      cudaGetLastError();
      set_error("cudaMalloc of %zu bytes of activations failed", need);
      return TETRIS_ERR_NOMEM;
    }
    hs.bytes = need;
  }
  float *d = static_cast<float *>(hs.ptr);
  float *d_in_nchw = d, *d_in_nhwc = d + in_elems, *d_out_nhwc = d + 2 * in_elems,
        *d_out_nchw = d + 2 * in_elems + out_elems;
  cudaStream_t st = hs.stream;
  TETRIS_CUDA_TRY(cudaMemcpyAsync(d_in_nchw, h_input_nchw, in_elems * sizeof(float), cudaMemcpyHostToDevice, st));
  if ((rc = launch_nchw_to_nhwc(d_in_nchw, d_in_nhwc, s.N, s.IC, s.H, s.W, st))) return rc;
  if ((rc = dispatch(f, d_in_nhwc, d_out_nhwc, s, st, TETRIS_VARIANT_AUTO))) return rc;
  if ((rc = launch_nhwc_to_nchw(d_out_nhwc, d_out_nchw, s.N, s.OC, s.OH, s.OW, st))) return rc;
  TETRIS_CUDA_TRY(cudaMemcpyAsync(h_output_nchw, d_out_nchw, out_elems * sizeof(float), cudaMemcpyDeviceToHost, st));
  return TETRIS_OK;
}

int tetris_host_sync(int device, int slot) {
  if (device < 0 || device >= kMaxWsDevices || slot >= kSlots) { set_error("bad device/slot"); return TETRIS_ERR_INVALID; }
  DeviceGuard guard(device);
  for (int i = 0; i < kSlots; ++i) {
    if (slot >= 0 && i != slot) continue;
    HostSlot &hs = g_slots[device][i];
    std::lock_guard<std::mutex> lock(hs.mutex);
    if (hs.stream && cudaStreamSynchronize(hs.stream) != cudaSuccess) {
      set_error("pipelined convolution failed: %s", cudaGetErrorString(cudaGetLastError()));
      return TETRIS_ERR_CUDA;
    }
  }
  return TETRIS_OK;
}

void tetris_release_workspace(void) {
  int prev = -1;
  cudaGetDevice(&prev);
  for (int dev = 0; dev < kMaxWsDevices; ++dev) {
    Workspace &ws = g_workspace[dev];
    std::lock_guard<std::mutex> lock(ws.mutex);
    if (!ws.ptr) continue;
    if (cudaSetDevice(dev) == cudaSuccess) cudaFree(ws.ptr);
    ws.ptr = nullptr;
    ws.bytes = 0;
  }
  for (int dev = 0; dev < kMaxWsDevices; ++dev)
    for (int i = 0; i < kSlots; ++i) {
      HostSlot &hs = g_slots[dev][i];
      std::lock_guard<std::mutex> lock(hs.mutex);
      if (!hs.stream && !hs.ptr) continue;
      if (cudaSetDevice(dev) != cudaSuccess) continue;
      if (hs.stream) { cudaStreamSynchronize(hs.stream); cudaStreamDestroy(hs.stream); }
      cudaFree(hs.ptr);
      hs.stream = nullptr; hs.ptr = nullptr; hs.bytes = 0;
    }
  if (prev >= 0) cudaSetDevice(prev);
}

int tetris_batch_slice(int batch_size, int world, int rank, int *begin, int *count) {
  if (batch_size < 0 || world < 1 || rank < 0 || rank >= world || !begin || !count) {
    set_error("bad slice arguments: batch=%d world=%d rank=%d", batch_size, world, rank);
    return TETRIS_ERR_INVALID;
  }
  const int base = batch_size / world, extra = batch_size % world;
  *begin = rank * base + (rank < extra ? rank : extra);
  *count = base + (rank < extra ? 1 : 0);
  return TETRIS_OK;
}

int tetris_conv2d_host_sharded(tetris_filter_t *const *filters, int n_gpus,
                               const float *h_input_nchw, float *h_output_nchw,
                               int batch_size, int img_h, int img_w, int stride, int padding) {
  if (!filters || n_gpus < 1) { set_error("bad shard arguments"); return TETRIS_ERR_INVALID; }
  for (int g = 0; g < n_gpus; ++g) {
    if (!filters[g]) { set_error("filters[%d] is NULL", g); return TETRIS_ERR_INVALID; }
    if (filters[g]->in_channel != filters[0]->in_channel ||
        filters[g]->out_channel != filters[0]->out_channel ||
        filters[g]->kernel_size != filters[0]->kernel_size || filters[g]->groups != filters[0]->groups) {
      set_error("filters[%d] has a different shape than filters[0]", g);
      return TETRIS_ERR_INVALID;
    }
  }
  ConvShape s;
  int rc = make_shape(filters[0], batch_size, img_h, img_w, stride, padding, &s);
  if (rc) return rc;
  if (batch_size > 0 && (!h_input_nchw || !h_output_nchw)) { set_error("input or output pointer is NULL"); return TETRIS_ERR_INVALID; }
  const size_t in_img = (size_t)s.IC * s.H * s.W, out_img = (size_t)s.OC * s.OH * s.OW;
  std::vector<int> status(n_gpus, TETRIS_OK);
  std::vector<std::string> messages(n_gpus);
  std::vector<std::thread> workers;
  for (int g = 0; g < n_gpus; ++g) {
    workers.emplace_back([&, g]() {
      int begin = 0, count = 0;
      tetris_batch_slice(batch_size, n_gpus, g, &begin, &count);
      if (count == 0) return;
      status[g] = tetris_conv2d_host(filters[g], h_input_nchw + (size_t)begin * in_img,
                                     h_output_nchw + (size_t)begin * out_img, count, img_h, img_w,
                                     stride, padding, nullptr);
      if (status[g]) messages[g] = tetris_last_error();
    });
  }
  for (auto &w : workers) w.join();
  for (int g = 0; g < n_gpus; ++g)
    if (status[g]) {
      set_error("shard %d: %s", g, messages[g].c_str());
      return status[g];
    }
  return TETRIS_OK;
}

int tetris_device_info(int device, int *sm_count, int *sm_clock_khz, int *fp32_lanes_per_sm) {
  int v = 0;
  if (sm_count) { TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device)); *sm_count = v; }
  if (sm_clock_khz) { TETRIS_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device)); *sm_clock_khz = v; }
  if (fp32_lanes_per_sm) *fp32_lanes_per_sm = 128;  // sm_100: 4 sub-partitions x 32 FP32 lanes
  return TETRIS_OK;
}

}  // extern "C"
