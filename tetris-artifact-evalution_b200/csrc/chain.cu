// Layer chains: the conv layers of a model run back to back on the device -- every layer reads
// the NHWC activations the previous one left in HBM, ReLU is applied at the convolution's own
// store (tensor-core variants) and 2x2 max-pooling by a small kernel in between -- eagerly on a
// stream, or captured once into a CUDA graph and replayed.
//
// The reference times isolated layers and adds the times up per model
// (evalution/overall_speedup.py:159-165); it has no chained execution.  The chain is the first
// step from "sum of isolated layers" to a forward pass: no per-layer host work, no layout
// conversion and no host round trip between layers.
#include <new>
#include <vector>

#include "internal.h"

namespace tetris {
namespace {

// y = max(y, 0) in place (for kernels whose store does not rectify itself)
__global__ void __launch_bounds__(256) relu_kernel(float *__restrict__ y, size_t n4, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) {
    float4 v = reinterpret_cast<float4 *>(y)[i];
    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
    reinterpret_cast<float4 *>(y)[i] = v;
  }
  if (i == 0)
    for (size_t j = n4 * 4; j < n; ++j) y[j] = fmaxf(y[j], 0.f);
}

// 2x2 max-pooling, stride 2, NHWC; odd trailing rows / columns are dropped (floor), as the
// networks' own pooling layers do.
__global__ void __launch_bounds__(256)
pool2x2_kernel(const float *__restrict__ in, float *__restrict__ out, int N, int H, int W, int C) {
  const int OH = H / 2, OW = W / 2;
  const size_t total = (size_t)N * OH * OW * C;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % C);
  size_t r = i / C;
  const int ow = (int)(r % OW); r /= OW;
  const int oh = (int)(r % OH);
  const int n = (int)(r / OH);
  const float *p = in + (((size_t)n * H + 2 * oh) * W + 2 * ow) * C + c;
  const size_t row = (size_t)W * C;
  out[i] = fmaxf(fmaxf(p[0], p[C]), fmaxf(p[row], p[row + C]));
}

}  // namespace

int launch_relu_inplace(float *y, size_t n, cudaStream_t st) {
  if (n == 0) return TETRIS_OK;
  const bool vec = (reinterpret_cast<uintptr_t>(y) & 15) == 0;
  const size_t n4 = vec ? n / 4 : 0;
  const size_t threads = n4 ? n4 : 1;
  relu_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(y, n4, n);
  TETRIS_CUDA_TRY(cudaGetLastError());
  return TETRIS_OK;
}

}  // namespace tetris

using namespace tetris;

struct tetris_chain {
  int device = 0, batch = 0;
  std::vector<tetris_chain_layer_t> layers;
  std::vector<ConvShape> shapes;      // conv shape of every layer
  std::vector<float *> conv_out;      // output of layer i (device, owned)
  std::vector<float *> pool_out;      // pooled output of layer i (owned; nullptr without pooling)
  int out_h = 0, out_w = 0, out_c = 0;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  const float *captured_in = nullptr;
};

extern "C" {

void tetris_chain_destroy(tetris_chain_t *c) {
  if (!c) return;
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(c->device);
  if (c->exec) cudaGraphExecDestroy(c->exec);
  if (c->graph) cudaGraphDestroy(c->graph);
  for (float *p : c->conv_out) cudaFree(p);
  for (float *p : c->pool_out) cudaFree(p);
  if (prev >= 0) cudaSetDevice(prev);
  delete c;
}

int tetris_chain_create(const tetris_chain_layer_t *layers, int n_layers, int batch_size, int img_h, int img_w,
                        tetris_chain_t **out) {
  if (!layers || !out || n_layers < 1 || batch_size < 1 || img_h < 1 || img_w < 1) {
    set_error("bad chain arguments");
    return TETRIS_ERR_INVALID;
  }
  *out = nullptr;
  tetris_chain *c = new (std::nothrow) tetris_chain();
  if (!c) { set_error("out of host memory"); return TETRIS_ERR_NOMEM; }
  c->batch = batch_size;
  int h = img_h, w = img_w, ch = -1, prev = -1;
  auto fail = [&](int code) { tetris_chain_destroy(c); if (prev >= 0) cudaSetDevice(prev); return code; };
  for (int i = 0; i < n_layers; ++i) {
    const tetris_chain_layer_t &l = layers[i];
    const tetris_filter *f = l.filter;
    if (!f) { set_error("layer %d has no filter", i); return fail(TETRIS_ERR_INVALID); }
    if (i == 0) {
      c->device = f->device;
      cudaGetDevice(&prev);
      if (cudaSetDevice(c->device) != cudaSuccess) { set_error("cudaSetDevice(%d) failed", c->device); return fail(TETRIS_ERR_CUDA); }
    }
    if (f->device != c->device) { set_error("layer %d lives on another device", i); return fail(TETRIS_ERR_INVALID); }
    if (ch >= 0 && f->in_channel != ch) {
      set_error("layer %d takes %d channels, the layer before it produces %d", i, f->in_channel, ch);
      return fail(TETRIS_ERR_INVALID);
    }
    if (l.stride < 1 || l.padding < 0 || h + 2 * l.padding < f->kernel_size || w + 2 * l.padding < f->kernel_size ||
        !(l.pool == 0 || l.pool == 2)) {
      set_error("layer %d: bad stride, padding or pooling for a %dx%d input", i, h, w);
      return fail(TETRIS_ERR_INVALID);
    }
    ConvShape s;
    s.N = batch_size; s.H = h; s.W = w; s.IC = f->in_channel; s.OC = f->out_channel; s.KS = f->kernel_size;
    s.S = l.stride; s.P = l.padding;
    s.OH = (h + 2 * l.padding - f->kernel_size) / l.stride + 1;
    s.OW = (w + 2 * l.padding - f->kernel_size) / l.stride + 1;
    s.relu = l.relu ? 1 : 0;
    c->shapes.push_back(s);
    c->layers.push_back(l);
    float *buf = nullptr, *pbuf = nullptr;
    const size_t elems = (size_t)batch_size * s.OH * s.OW * s.OC;
    if (cudaMalloc(&buf, elems * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      set_error("cudaMalloc of %zu bytes of activations failed", elems * sizeof(float));
      return fail(TETRIS_ERR_NOMEM);
    }
    c->conv_out.push_back(buf);
    h = s.OH; w = s.OW; ch = s.OC;
    if (l.pool == 2) {
      if (h < 2 || w < 2) { cudaFree(buf); c->conv_out.pop_back(); set_error("layer %d: nothing left to pool", i); return fail(TETRIS_ERR_INVALID); }
      h /= 2; w /= 2;
      if (cudaMalloc(&pbuf, (size_t)batch_size * h * w * ch * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        c->pool_out.push_back(nullptr);
        set_error("cudaMalloc of pooled activations failed");
        return fail(TETRIS_ERR_NOMEM);
      }
    }
    c->pool_out.push_back(pbuf);
  }
  c->out_h = h; c->out_w = w; c->out_c = ch;
  if (prev >= 0) cudaSetDevice(prev);
  *out = c;
  return TETRIS_OK;
}

int tetris_chain_output(const tetris_chain_t *c, const float **d_output_nhwc, int *h, int *w, int *channels) {
  if (!c) { set_error("chain handle is NULL"); return TETRIS_ERR_INVALID; }
  const size_t last = c->layers.size() - 1;
  if (d_output_nhwc) *d_output_nhwc = c->pool_out[last] ? c->pool_out[last] : c->conv_out[last];
  if (h) *h = c->out_h;
  if (w) *w = c->out_w;
  if (channels) *channels = c->out_c;
  return TETRIS_OK;
}

int tetris_chain_download(const tetris_chain_t *c, float *h_output_nhwc, size_t capacity) {
  if (!c || !h_output_nhwc) { set_error("chain handle or output is NULL"); return TETRIS_ERR_INVALID; }
  const size_t n = (size_t)c->batch * c->out_h * c->out_w * c->out_c, last = c->layers.size() - 1;
  if (capacity < n) { set_error("output buffer too small: %zu floats for %zu", capacity, n); return TETRIS_ERR_INVALID; }
  int prev = -1;
  TETRIS_CUDA_TRY(cudaGetDevice(&prev));
  TETRIS_CUDA_TRY(cudaSetDevice(c->device));
  const float *src = c->pool_out[last] ? c->pool_out[last] : c->conv_out[last];
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(h_output_nhwc, src, n * sizeof(float), cudaMemcpyDeviceToHost);
  cudaSetDevice(prev);
  if (e != cudaSuccess) { set_error("download of the chain's output failed: %s", cudaGetErrorString(e)); return TETRIS_ERR_CUDA; }
  return TETRIS_OK;
}

int tetris_chain_run(tetris_chain_t *c, const float *d_input_nhwc, void *stream) {
  if (!c || !d_input_nhwc) { set_error("chain handle or input is NULL"); return TETRIS_ERR_INVALID; }
  cudaStream_t st = (cudaStream_t)stream;
  const float *x = d_input_nhwc;
  for (size_t i = 0; i < c->layers.size(); ++i) {
    const ConvShape &s = c->shapes[i];
    int rc = conv_dispatch_auto(c->layers[i].filter, x, c->conv_out[i], s, st);
    if (rc) return rc;
    x = c->conv_out[i];
    if (c->pool_out[i]) {
      const size_t total = (size_t)s.N * (s.OH / 2) * (s.OW / 2) * s.OC;
      pool2x2_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(x, c->pool_out[i], s.N, s.OH, s.OW, s.OC);
      TETRIS_CUDA_TRY(cudaGetLastError());
      x = c->pool_out[i];
    }
  }
  return TETRIS_OK;
}

int tetris_chain_capture(tetris_chain_t *c, const float *d_input_nhwc) {
  if (!c || !d_input_nhwc) { set_error("chain handle or input is NULL"); return TETRIS_ERR_INVALID; }
  int prev = -1;
  TETRIS_CUDA_TRY(cudaGetDevice(&prev));
  TETRIS_CUDA_TRY(cudaSetDevice(c->device));
  if (c->exec) { cudaGraphExecDestroy(c->exec); c->exec = nullptr; }
  if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; }
  cudaStream_t st = nullptr;
  auto done = [&](int code) { if (st) cudaStreamDestroy(st); cudaSetDevice(prev); return code; };
  if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) { set_error("cudaStreamCreate failed"); return done(TETRIS_ERR_CUDA); }
  // once eagerly: every layer plans its launch (tile shapes, tensor maps) outside the capture
  int rc = tetris_chain_run(c, d_input_nhwc, st);
  if (rc) return done(rc);
  if (cudaStreamSynchronize(st) != cudaSuccess) { set_error("chain run failed: %s", cudaGetErrorString(cudaGetLastError())); return done(TETRIS_ERR_CUDA); }
  if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { set_error("cudaStreamBeginCapture failed"); return done(TETRIS_ERR_CUDA); }
  rc = tetris_chain_run(c, d_input_nhwc, st);
  const cudaError_t e = cudaStreamEndCapture(st, &c->graph);
  if (rc) { if (c->graph) { cudaGraphDestroy(c->graph); c->graph = nullptr; } return done(rc); }
  if (e != cudaSuccess || cudaGraphInstantiate(&c->exec, c->graph, 0) != cudaSuccess) {
    set_error("capturing the chain into a CUDA graph failed: %s", cudaGetErrorString(cudaGetLastError()));
    return done(TETRIS_ERR_CUDA);
  }
  c->captured_in = d_input_nhwc;
  return done(TETRIS_OK);
}

int tetris_chain_replay(tetris_chain_t *c, void *stream) {
  if (!c || !c->exec) { set_error("the chain has not been captured"); return TETRIS_ERR_INVALID; }
  TETRIS_CUDA_TRY(cudaGraphLaunch(c->exec, (cudaStream_t)stream));
  return TETRIS_OK;
}

}  // extern "C"
