// Compressed-filter files: tetris_filter_save / tetris_filter_load / tetris_filter_file_check.
//
// The reference rebuilds its SparseFilter -- an O(nnz^2) host reorder followed by five blocking
// uploads (Tetris/spconv2d_utils.h:99-264) -- for every tile configuration it times
// (Tetris/spconv2d.cc:285-311), and again in every process.  Here the compressed forms are
// written once and read back: the LIST and PROGRAM forms as they lie on the device, the tile
// plans chosen by tetris_conv2d_tune for the shapes tuned so far, and for a depthwise filter
// the dense taps.  The tensor-core tile images are not stored (they are dense: 8 bytes per
// weight position, zeros included); the loader rebuilds them on the device from the LIST form.
//
// File layout, little-endian, no padding between parts:
//   FileHeader                                  (fixed size, see below)
//   int32  list_offsets[P + 1], prog_offsets[P + 1]          P = n_oc_blocks * n_stages
//   uint64 lists[n_list_units], ops[n_ops]
//   float  dense[OC * KS * KS]                                depthwise filters only (then P = 0)
//   int32  tuned[n_tuned][kTunedInts]                         see tiled_plans_export
// `checksum` is FNV-1a (64 bit) over everything after the header.
#include <stdio.h>
#include <string.h>

#include <vector>

#include "internal.h"

namespace tetris {
namespace {

constexpr char kMagic[8] = {'T', 'E', 'T', 'R', 'I', 'S', 'F', '1'};
constexpr uint32_t kVersion = 1;

struct FileHeader {
  char magic[8];
  uint32_t version;
  uint32_t header_bytes;
  int32_t in_channel, out_channel, kernel_size, groups;
  int32_t oc_block, tile_ic, n_oc_blocks, n_stages;
  int32_t max_prog_ops, max_list_units, deterministic, n_tuned;
  int64_t nnz, n_ops, n_list_units;
  uint64_t payload_bytes;
  uint64_t checksum;
};

uint64_t fnv1a(const unsigned char *p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  return h;
}

// Sizes of the parts the header promises; false when the header is inconsistent.
bool payload_layout(const FileHeader &h, size_t *offsets_bytes, size_t *lists_bytes, size_t *ops_bytes,
                    size_t *dense_bytes, size_t *tuned_bytes) {
  if (h.in_channel < 1 || h.out_channel < 1 || h.kernel_size < 1 || h.kernel_size > 8) return false;
  if (h.n_tuned < 0 || h.n_tuned > 64) return false;
  *tuned_bytes = (size_t)h.n_tuned * kTunedInts * sizeof(int32_t);
  if (h.groups != 1) {
    if (h.groups != h.in_channel || h.groups != h.out_channel) return false;
    if (h.n_oc_blocks != 0 || h.n_stages != 0 || h.n_ops != 0 || h.n_list_units != 0) return false;
    *offsets_bytes = *lists_bytes = *ops_bytes = 0;
    *dense_bytes = (size_t)h.out_channel * h.kernel_size * h.kernel_size * sizeof(float);
    return true;
  }
  if (!(h.oc_block == 8 || h.oc_block == 16) || h.tile_ic < 4 || h.tile_ic > kMaxTileIc || (h.tile_ic & 3)) return false;
  if (h.n_oc_blocks != (h.out_channel + h.oc_block - 1) / h.oc_block) return false;
  if (h.n_stages != (h.in_channel + h.tile_ic - 1) / h.tile_ic) return false;
  const int64_t P = (int64_t)h.n_oc_blocks * h.n_stages;
  if (h.n_ops < kTailPadOps || h.n_list_units < 2 || h.n_ops > (1ll << 31) || h.n_list_units > (1ll << 31)) return false;
  if (h.nnz < 0 || h.nnz > (int64_t)h.out_channel * h.in_channel * h.kernel_size * h.kernel_size) return false;
  *offsets_bytes = (size_t)(P + 1) * sizeof(int32_t);
  *lists_bytes = (size_t)h.n_list_units * sizeof(uint64_t);
  *ops_bytes = (size_t)h.n_ops * sizeof(uint64_t);
  *dense_bytes = 0;
  return true;
}

// Reads and validates a whole file.  On success `payload` holds everything after the header.
int read_file(const char *path, FileHeader *h, std::vector<unsigned char> *payload) {
  if (!path) { set_error("path is NULL"); return TETRIS_ERR_INVALID; }
  FILE *fp = fopen(path, "rb");
  if (!fp) { set_error("cannot open %s", path); return TETRIS_ERR_INVALID; }
  auto fail = [&](const char *what) {
    fclose(fp);
    set_error("%s: %s", path, what);
    return TETRIS_ERR_INVALID;
  };
  if (fread(h, 1, sizeof(*h), fp) != sizeof(*h)) return fail("shorter than a filter-file header");
  if (memcmp(h->magic, kMagic, sizeof(kMagic)) != 0) return fail("not a compressed-filter file (bad magic)");
  if (h->version != kVersion || h->header_bytes != sizeof(FileHeader)) return fail("unknown filter-file version");
  size_t ob = 0, lb = 0, pb = 0, db = 0, tb = 0;
  if (!payload_layout(*h, &ob, &lb, &pb, &db, &tb)) return fail("inconsistent header fields");
  const size_t want = 2 * ob + lb + pb + db + tb;
  if (h->payload_bytes != want) return fail("payload size does not match the header fields");
  payload->resize(want);
  if (want && fread(payload->data(), 1, want, fp) != want) return fail("truncated: payload shorter than the header says");
  unsigned char extra;
  if (fread(&extra, 1, 1, fp) == 1) return fail("trailing bytes after the payload");
  fclose(fp);
  if (fnv1a(payload->data(), payload->size()) != h->checksum) {
    set_error("%s: checksum mismatch (corrupt file)", path);
    return TETRIS_ERR_INVALID;
  }
  if (h->groups == 1) {
    // offsets must be non-decreasing, even, and end where the streams end
    const int64_t P = (int64_t)h->n_oc_blocks * h->n_stages;
    const int32_t *lo = reinterpret_cast<const int32_t *>(payload->data());
    const int32_t *po = lo + (P + 1);
    for (int64_t i = 0; i <= P; ++i) {
      if (lo[i] < 0 || po[i] < 0 || (i && (lo[i] < lo[i - 1] || po[i] < po[i - 1])) || (lo[i] & 1) || (po[i] & 1)) {
        set_error("%s: piece offsets are not a non-decreasing even sequence", path);
        return TETRIS_ERR_INVALID;
      }
      if (i && (lo[i] - lo[i - 1] > h->max_list_units || po[i] - po[i - 1] > h->max_prog_ops)) {
        set_error("%s: a piece is longer than the header's maximum", path);
        return TETRIS_ERR_INVALID;
      }
    }
    if (lo[0] != 0 || po[0] != 0 || (int64_t)lo[P] + 2 != h->n_list_units || (int64_t)po[P] + kTailPadOps != h->n_ops) {
      set_error("%s: piece offsets do not end where the record streams end", path);
      return TETRIS_ERR_INVALID;
    }
  }
  return TETRIS_OK;
}

// LIST form -> dense OIHW (zeroed by the caller): one warp per piece, as in the compressor.
__global__ void __launch_bounds__(256)
lists_to_dense_kernel(const uint64_t *__restrict__ units, const int32_t *__restrict__ offsets, float *__restrict__ dense,
                      int IC, int OC, int KS, int K, int TIC, int B, int T) {
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (p >= B * T) return;
  const int b = p / T, t = p - b * T;
  const uint32_t *hdr = reinterpret_cast<const uint32_t *>(units + offsets[p]);
  long long pos = (long long)offsets[p] + list_header_units(K);
  for (int k = 0; k < K; ++k) {
    const int n_k = (int)hdr[k], oc = b * K + k;
    for (int i = lane; i < n_k; i += 32) {
      const uint64_t u = units[pos + i];
      const uint32_t code = (uint32_t)(u >> 32), icl = code >> 8, r = (code >> 4) & 15u, s = code & 15u;
      const int ic = t * TIC + (int)icl;
      if ((int)icl < TIC && ic < IC && oc < OC && (int)r < KS && (int)s < KS)  // (padding records point at channel TIC)
        dense[(((size_t)oc * IC + ic) * KS + r) * KS + s] = __uint_as_float((uint32_t)u);
    }
    pos += n_k;
  }
}

}  // namespace
}  // namespace tetris

using namespace tetris;

extern "C" {

int tetris_filter_save(const tetris_filter_t *f, const char *path) {
  if (!f || !path) { set_error("filter handle or path is NULL"); return TETRIS_ERR_INVALID; }
  int prev = -1;
  TETRIS_CUDA_TRY(cudaGetDevice(&prev));
  TETRIS_CUDA_TRY(cudaSetDevice(f->device));
  FileHeader h;
  memset(&h, 0, sizeof(h));
  memcpy(h.magic, kMagic, sizeof(kMagic));
  h.version = kVersion; h.header_bytes = sizeof(FileHeader);
  h.in_channel = f->in_channel; h.out_channel = f->out_channel; h.kernel_size = f->kernel_size; h.groups = f->groups;
  h.oc_block = f->oc_block; h.tile_ic = f->tile_ic; h.n_oc_blocks = f->n_oc_blocks; h.n_stages = f->n_stages;
  h.max_prog_ops = f->max_prog_ops; h.max_list_units = f->max_list_units; h.deterministic = f->deterministic;
  h.nnz = f->nnz; h.n_ops = f->n_ops; h.n_list_units = f->n_list_units;
  std::vector<int32_t> tuned;
  tiled_plans_export(f, &tuned);
  h.n_tuned = (int32_t)(tuned.size() / kTunedInts);
  size_t ob = 0, lb = 0, pb = 0, db = 0, tb = 0;
  if (!payload_layout(h, &ob, &lb, &pb, &db, &tb)) { cudaSetDevice(prev); set_error("filter handle is inconsistent"); return TETRIS_ERR_INVALID; }
  std::vector<unsigned char> payload(2 * ob + lb + pb + db + tb);
  unsigned char *w = payload.data();
  cudaError_t err = cudaSuccess;
  auto pull = [&](const void *src, size_t n) {
    if (n && err == cudaSuccess) err = cudaMemcpy(w, src, n, cudaMemcpyDeviceToHost);
    w += n;
  };
  pull(f->d_list_offsets, ob); pull(f->d_prog_offsets, ob); pull(f->d_lists, lb); pull(f->d_ops, pb); pull(f->d_dense, db);
  cudaSetDevice(prev);
  if (err != cudaSuccess) { set_error("copy of the compressed filter to the host failed: %s", cudaGetErrorString(err)); return TETRIS_ERR_CUDA; }
  if (tb) memcpy(w, tuned.data(), tb);
  h.payload_bytes = payload.size();
  h.checksum = fnv1a(payload.data(), payload.size());
  FILE *fp = fopen(path, "wb");
  if (!fp) { set_error("cannot create %s", path); return TETRIS_ERR_INVALID; }
  const bool ok = fwrite(&h, 1, sizeof(h), fp) == sizeof(h) &&
                  (payload.empty() || fwrite(payload.data(), 1, payload.size(), fp) == payload.size());
  if (fclose(fp) != 0 || !ok) { set_error("write to %s failed", path); return TETRIS_ERR_INVALID; }
  return TETRIS_OK;
}

int tetris_filter_file_check(const char *path, tetris_filter_info_t *info) {
  FileHeader h;
  std::vector<unsigned char> payload;
  const int rc = read_file(path, &h, &payload);
  if (rc) return rc;
  if (info) {
    memset(info, 0, sizeof(*info));
    info->in_channel = h.in_channel; info->out_channel = h.out_channel; info->kernel_size = h.kernel_size;
    info->groups = h.groups; info->oc_block = h.oc_block; info->tile_ic = h.tile_ic;
    info->n_oc_blocks = h.n_oc_blocks; info->n_stages = h.n_stages;
    info->nnz = h.nnz; info->n_ops = h.n_ops; info->n_list_units = h.n_list_units;
    info->compressed_bytes = (int64_t)h.payload_bytes;
    info->device = -1;
  }
  return TETRIS_OK;
}

int tetris_filter_load(const char *path, int device, tetris_filter_t **out) {
  if (!out) { set_error("out pointer is NULL"); return TETRIS_ERR_INVALID; }
  *out = nullptr;
  FileHeader h;
  std::vector<unsigned char> payload;
  int rc = read_file(path, &h, &payload);
  if (rc) return rc;
  int n_dev = 0, prev = -1;
  TETRIS_CUDA_TRY(cudaGetDeviceCount(&n_dev));
  if (device < 0 || device >= n_dev) { set_error("device %d out of range (%d visible)", device, n_dev); return TETRIS_ERR_INVALID; }
  TETRIS_CUDA_TRY(cudaGetDevice(&prev));
  TETRIS_CUDA_TRY(cudaSetDevice(device));
  tetris_filter *f = new (std::nothrow) tetris_filter();
  if (!f) { cudaSetDevice(prev); set_error("out of host memory"); return TETRIS_ERR_NOMEM; }
  memset(f, 0, sizeof(*f));
  f->in_channel = h.in_channel; f->out_channel = h.out_channel; f->kernel_size = h.kernel_size; f->groups = h.groups;
  f->oc_block = h.oc_block; f->tile_ic = h.tile_ic; f->n_oc_blocks = h.n_oc_blocks; f->n_stages = h.n_stages;
  f->max_prog_ops = h.max_prog_ops; f->max_list_units = h.max_list_units; f->deterministic = h.deterministic;
  f->nnz = h.nnz; f->n_ops = h.n_ops; f->n_list_units = h.n_list_units; f->device = device;
  f->plan_cache = tiled_plan_cache_new();
  size_t ob = 0, lb = 0, pb = 0, db = 0, tb = 0;
  payload_layout(h, &ob, &lb, &pb, &db, &tb);
  const unsigned char *r = payload.data();
  float *d_dense = nullptr;
  auto fail = [&](int code) {
    cudaFree(d_dense);
    tetris_filter_destroy(f);
    cudaSetDevice(prev);
    return code;
  };
  cudaError_t err = cudaSuccess;
  auto push = [&](void **dst, size_t n) {
    if (n && err == cudaSuccess) err = cudaMalloc(dst, n);
    if (n && err == cudaSuccess) err = cudaMemcpy(*dst, r, n, cudaMemcpyHostToDevice);
    r += n;
  };
  push((void **)&f->d_list_offsets, ob); push((void **)&f->d_prog_offsets, ob);
  push((void **)&f->d_lists, lb); push((void **)&f->d_ops, pb); push((void **)&f->d_dense, db);
  if (err != cudaSuccess) {
    cudaGetLastError();
    set_error("upload of the compressed filter failed: %s", cudaGetErrorString(err));
    return fail(err == cudaErrorMemoryAllocation ? TETRIS_ERR_NOMEM : TETRIS_ERR_CUDA);
  }
  if (f->groups == 1) {
    // the tensor-core tile images: back to dense on the device, then as at creation
    const size_t dense_bytes = (size_t)f->out_channel * f->in_channel * f->kernel_size * f->kernel_size * sizeof(float);
    if (cudaMalloc(&d_dense, dense_bytes) != cudaSuccess) {
      cudaGetLastError();
      set_error("cudaMalloc of %zu bytes for the dense filter failed", dense_bytes);
      return fail(TETRIS_ERR_NOMEM);
    }
    cudaMemset(d_dense, 0, dense_bytes);
    const int P = f->n_oc_blocks * f->n_stages;
    lists_to_dense_kernel<<<(P + 7) / 8, 256>>>(f->d_lists, f->d_list_offsets, d_dense, f->in_channel, f->out_channel,
                                                 f->kernel_size, f->oc_block, f->tile_ic, f->n_oc_blocks, f->n_stages);
    if ((rc = conv_tc_prepare(f, d_dense)) || (rc = conv_tc16_prepare(f, d_dense))) return fail(rc);
    if (cudaDeviceSynchronize() != cudaSuccess) {
      set_error("rebuilding the tensor-core tile images failed: %s", cudaGetErrorString(cudaGetLastError()));
      return fail(TETRIS_ERR_CUDA);
    }
    cudaFree(d_dense);
    d_dense = nullptr;
    if (tb) tiled_plans_import(f, reinterpret_cast<const int32_t *>(r), h.n_tuned);
  }
  cudaSetDevice(prev);
  *out = f;
  return TETRIS_OK;
}

}  // extern "C"
