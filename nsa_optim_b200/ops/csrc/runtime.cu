// Library runtime: error text, launch counter, kernel status block, tensor-map encoder.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "host.cuh"

namespace {
thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};
KernelStatus* g_status[64] = {nullptr};
int g_sms[64] = {0};
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn encoder() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

namespace nsa {
int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
  return NSA_ERR_CUDA;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

KernelStatus* status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    KernelStatus* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(KernelStatus), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
      return nullptr;
    memset(h, 0, sizeof(KernelStatus));
    g_status[dev] = h;   // unified addressing: the host pointer is valid on the device
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sms[dev] = n > 0 ? n : 148;
  }
  return g_sms[dev];
}

// Driver-API calls need a context current on the calling thread.  Threads that have only been
// handed a device index (autograd worker threads) get the primary context bound here.
static void bind_primary_context() {
  static thread_local bool bound = false;
  if (bound) return;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaSetDevice(dev);
  cudaFree(nullptr);
  bound = true;
}

int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  bind_primary_context();
  EncodeTiledFn enc = encoder();
  if (!enc) return fail(NSA_ERR_DRIVER_API, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gd[5], gs[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gs[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gd, gs, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[200];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu)", (int)r, rank,
             (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 1));
    return fail(NSA_ERR_DRIVER_API, msg);
  }
  return 0;
}

int make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                     uint32_t box_inner, uint32_t box_outer) {
  bind_primary_context();
  EncodeTiledFn enc = encoder();
  if (!enc) return fail(NSA_ERR_DRIVER_API, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gd[2] = {inner, outer}, gs[1] = {ld * 4};
  cuuint32_t bx[2] = {box_inner, box_outer}, es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gd, gs, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[160];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled (fp32) failed with CUresult %d (%llu x %llu)", (int)r,
             (unsigned long long)inner, (unsigned long long)outer);
    return fail(NSA_ERR_DRIVER_API, msg);
  }
  return 0;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {ld * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tmap_bf16(out, base, 2, dims, strides, box, 1);
}
}  // namespace nsa

extern "C" const char* nsa_last_error() { return g_err; }
extern "C" long long nsa_launch_count() { return g_launches.load(); }
extern "C" void nsa_launch_count_reset() { g_launches.store(0); }
// out[4] = {code, block, info, count}; reset clears the block after reading.
extern "C" int nsa_status_read(int* out, int reset) {
  KernelStatus* s = nsa::status_ptr();
  if (!s) return NSA_ERR_CUDA;
  out[0] = s->code; out[1] = s->block; out[2] = s->info; out[3] = s->count;
  if (reset) memset(s, 0, sizeof(KernelStatus));
  return 0;
}
extern "C" int nsa_sm_count() { return nsa::sm_count(); }

// Row-pitched device-to-device copy (column slices of row-major matrices) on `st`.
extern "C" int nsa_copy2d(void* dst, long dst_pitch_bytes, const void* src, long src_pitch_bytes, long width_bytes, long rows,
                          cudaStream_t st) {
  if (rows <= 0 || width_bytes <= 0) return 0;
  cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch_bytes), src, static_cast<size_t>(src_pitch_bytes),
                                    static_cast<size_t>(width_bytes), static_cast<size_t>(rows), cudaMemcpyDeviceToDevice, st);
  return e == cudaSuccess ? 0 : nsa::fail_cuda(e, "nsa_copy2d");
}
