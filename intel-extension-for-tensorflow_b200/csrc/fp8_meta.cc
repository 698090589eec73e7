// Save / restore of the FP8 delayed-scaling state (amax history, scale, scale_inv) as one self-describing host blob.
// In the reference this state lives in non-trainable tf.Variables (itex/python/transformer/base.py:60-93) and is saved
// and restored with the model's checkpoint; here it lives in three device arrays per layer, and these two calls are what
// a checkpoint writer / reader around this library uses.
#include <cstring>

#include "common.h"

namespace {
struct BlobHeader {
  uint32_t magic;    // 'I','F','8','M'
  uint32_t version;  // 1
  int32_t history_len;
  int32_t n;
};
constexpr uint32_t kMagic = 0x4D384649u;
size_t BlobBytes(int64_t hlen, int64_t n) { return sizeof(BlobHeader) + size_t(hlen * n + 2 * n) * sizeof(float); }
}  // namespace

using namespace itexb;

extern "C" size_t itexb_fp8_meta_blob_bytes(int32_t history_len, int32_t n) {
  return (history_len <= 0 || n <= 0) ? 0 : BlobBytes(history_len, n);
}

extern "C" int itexb_fp8_meta_save(const float* amax_history, const float* scale, const float* scale_inv, int32_t history_len, int32_t n,
                                   void* blob, size_t blob_bytes, itexb_stream_t stream) {
  ITEXB_REQUIRE(amax_history != nullptr && scale != nullptr && scale_inv != nullptr && blob != nullptr && history_len > 0 && n > 0,
                ITEXB_INVALID_ARGUMENT, "fp8_meta_save: bad arguments");
  ITEXB_REQUIRE(blob_bytes >= BlobBytes(history_len, n), ITEXB_INVALID_ARGUMENT, "fp8_meta_save: the blob needs %zu bytes, %zu given",
                BlobBytes(history_len, n), blob_bytes);
  BlobHeader h{kMagic, 1u, history_len, n};
  std::memcpy(blob, &h, sizeof(h));
  float* p = reinterpret_cast<float*>(static_cast<unsigned char*>(blob) + sizeof(h));
  cudaStream_t st = AsCuda(stream);
  // stream-ordered: the state saved is the state after everything queued on `stream` so far
  ITEXB_CUDA(cudaMemcpyAsync(p, amax_history, size_t(history_len) * n * sizeof(float), cudaMemcpyDeviceToHost, st));
  ITEXB_CUDA(cudaMemcpyAsync(p + size_t(history_len) * n, scale, size_t(n) * sizeof(float), cudaMemcpyDeviceToHost, st));
  ITEXB_CUDA(cudaMemcpyAsync(p + size_t(history_len) * n + n, scale_inv, size_t(n) * sizeof(float), cudaMemcpyDeviceToHost, st));
  ITEXB_CUDA(cudaStreamSynchronize(st));
  return ITEXB_OK;
}

extern "C" int itexb_fp8_meta_load(float* amax_history, float* scale, float* scale_inv, int32_t history_len, int32_t n, const void* blob,
                                   size_t blob_bytes, itexb_stream_t stream) {
  ITEXB_REQUIRE(amax_history != nullptr && scale != nullptr && scale_inv != nullptr && blob != nullptr, ITEXB_INVALID_ARGUMENT,
                "fp8_meta_load: NULL argument");
  ITEXB_REQUIRE(blob_bytes >= sizeof(BlobHeader), ITEXB_INVALID_ARGUMENT, "fp8_meta_load: the blob is shorter than its header");
  BlobHeader h;
  std::memcpy(&h, blob, sizeof(h));
  ITEXB_REQUIRE(h.magic == kMagic && h.version == 1u, ITEXB_INVALID_ARGUMENT, "fp8_meta_load: not an FP8 meta blob (magic %08x, version %u)", h.magic,
                h.version);
  ITEXB_REQUIRE(h.history_len == history_len && h.n == n, ITEXB_INVALID_ARGUMENT,
                "fp8_meta_load: the blob holds history %d x %d slots, the layer has %d x %d", h.history_len, h.n, history_len, n);
  ITEXB_REQUIRE(blob_bytes >= BlobBytes(history_len, n), ITEXB_INVALID_ARGUMENT, "fp8_meta_load: the blob is truncated");
  const float* p = reinterpret_cast<const float*>(static_cast<const unsigned char*>(blob) + sizeof(h));
  cudaStream_t st = AsCuda(stream);
  ITEXB_CUDA(cudaMemcpyAsync(amax_history, p, size_t(history_len) * n * sizeof(float), cudaMemcpyHostToDevice, st));
  ITEXB_CUDA(cudaMemcpyAsync(scale, p + size_t(history_len) * n, size_t(n) * sizeof(float), cudaMemcpyHostToDevice, st));
  ITEXB_CUDA(cudaMemcpyAsync(scale_inv, p + size_t(history_len) * n + n, size_t(n) * sizeof(float), cudaMemcpyHostToDevice, st));
  ITEXB_CUDA(cudaStreamSynchronize(st));  // the blob may be released by the caller on return
  return ITEXB_OK;
}
