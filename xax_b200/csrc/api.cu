// Context, status reporting and tensor-map construction for the C ABI.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace xaxb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

// On unless the environment says XAXB_PROGRAMMATIC_LAUNCH=0 (or xaxb_set_programmatic_launch(0)).
static bool pdl_default() {
  const char* v = getenv("XAXB_PROGRAMMATIC_LAUNCH");
  return !(v && v[0] == '0');
}
static bool g_pdl = pdl_default();
bool pdl_enabled() { return g_pdl; }
void set_pdl_enabled(bool on) { g_pdl = on; }

// Kernels launched by this library in this process (all contexts, all streams).
static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("%s: %s", what, cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  return XAXB_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static CUtensorMapDataType tmap_dtype(int elem_bytes) {
  return elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

// Row-major 2-D tensor [outer, inner]; 128-byte swizzle; out-of-range elements read as zero.
int make_tmap_2d(const Ctx* ctx, CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || box_inner * elem_bytes != 128 ||
      box_outer > 256 || box_outer == 0) {
    set_last_error("tensor map: base %p / row stride %llu must be 16-byte aligned, box %ux%u", base,
                   (unsigned long long)row_stride_bytes, box_inner, box_outer);
    return XAXB_BAD_ARGUMENT;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, tmap_dtype(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(2d) failed with CUresult %d", (int)r);
    return XAXB_LAUNCH_FAILED;
  }
  return XAXB_OK;
}

// The same tensor with an un-swizzled box: box rows lie back to back in shared memory, box_inner * elem_bytes
// apart (a multiple of 16 bytes).
int make_tmap_2d_plain(const Ctx* ctx, CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner,
                       uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || ((box_inner * elem_bytes) & 15) ||
      box_inner == 0 || box_inner > 256 || box_outer > 256 || box_outer == 0) {
    set_last_error("tensor map: base %p / row stride %llu must be 16-byte aligned, box %ux%u", base,
                   (unsigned long long)row_stride_bytes, box_inner, box_outer);
    return XAXB_BAD_ARGUMENT;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, tmap_dtype(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(2d, plain) failed with CUresult %d", (int)r);
    return XAXB_LAUNCH_FAILED;
  }
  return XAXB_OK;
}

int make_tmap_4d(const Ctx* ctx, CUtensorMap* map, const void* base, int elem_bytes, const uint64_t dims_in[4],
                 const uint64_t strides_bytes[3], const uint32_t box_in[4]) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || box_in[0] * elem_bytes != 128) {
    set_last_error("tensor map: base %p must be 16-byte aligned and the box 128 bytes wide", base);
    return XAXB_BAD_ARGUMENT;
  }
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) {
    dims[i] = dims_in[i];
    box[i] = box_in[i];
  }
  for (int i = 0; i < 3; ++i) {
    if (strides_bytes[i] & 15) {
      set_last_error("tensor map: stride %d = %llu bytes is not a multiple of 16", i,
                     (unsigned long long)strides_bytes[i]);
      return XAXB_BAD_ARGUMENT;
    }
    strides[i] = strides_bytes[i];
  }
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, tmap_dtype(elem_bytes), 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled(4d) failed with CUresult %d", (int)r);
    return XAXB_LAUNCH_FAILED;
  }
  return XAXB_OK;
}

}  // namespace xaxb

using namespace xaxb;

extern "C" {

int xaxb_ctx_create(int device, xaxb_ctx** out) {
  if (!out) return XAXB_BAD_ARGUMENT;
  *out = nullptr;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    set_last_error("cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    set_last_error("cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  if (prop.major != 10) {
    set_last_error("device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    return XAXB_UNSUPPORTED;
  }
  Ctx* c = new Ctx();
  c->device = device;
  c->num_sms = prop.multiProcessorCount;
  c->d_status = nullptr;
  c->encode_tiled = nullptr;
  cudaDriverEntryPointQueryResult q;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &c->encode_tiled, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !c->encode_tiled) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    delete c;
    return XAXB_UNSUPPORTED;
  }
  e = cudaMalloc(&c->d_status, kStatusBlockBytes);
  if (e == cudaSuccess) {
    unsigned long long block[kStatusBlockBytes / 8] = {0, kDefaultWaitLimitNs, kDefaultPeerWaitLimitNs, 0};
    e = cudaMemcpy(c->d_status, block, sizeof(block), cudaMemcpyHostToDevice);
  }
  if (e != cudaSuccess) {
    set_last_error("status word: %s", cudaGetErrorString(e));
    delete c;
    return XAXB_LAUNCH_FAILED;
  }
  *out = reinterpret_cast<xaxb_ctx*>(c);
  return XAXB_OK;
}

int xaxb_ctx_destroy(xaxb_ctx* ctx) {
  if (!ctx) return XAXB_OK;
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  cudaSetDevice(c->device);
  if (c->d_status) cudaFree(c->d_status);
  delete c;
  return XAXB_OK;
}

int xaxb_ctx_status(xaxb_ctx* ctx, void* stream, int* site) {
  if (!ctx) return XAXB_BAD_ARGUMENT;
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int host[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(host, c->d_status, sizeof(host), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    set_last_error("status read: %s", cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  if (site) *site = 0;
  if (host[0] == 0) return XAXB_OK;
  cudaMemsetAsync(c->d_status, 0, sizeof(host), s);
  // The word holds status * 1000 + site so one atomic records both.
  if (site) *site = host[0] % 1000;
  return host[0] / 1000;
}

int xaxb_num_sms(const xaxb_ctx* ctx) { return ctx ? reinterpret_cast<const Ctx*>(ctx)->num_sms : 0; }

const char* xaxb_status_string(int status) {
  switch (status) {
    case XAXB_OK: return "ok";
    case XAXB_BAD_ARGUMENT: return "bad argument";
    case XAXB_UNSUPPORTED: return "unsupported configuration";
    case XAXB_WORKSPACE_TOO_SMALL: return "workspace too small";
    case XAXB_LAUNCH_FAILED: return "CUDA launch or runtime failure";
    case XAXB_DEVICE_TIMEOUT: return "device-side wait timed out";
    case XAXB_CACHE_OVERFLOW: return "KV cache overflow";
    default: return "unknown status";
  }
}

const char* xaxb_last_error(void) { return g_last_error; }

int xaxb_set_programmatic_launch(int on) {
  xaxb::set_pdl_enabled(on != 0);
  return XAXB_OK;
}

int xaxb_programmatic_launch_enabled(void) { return xaxb::pdl_enabled() ? 1 : 0; }

long long xaxb_launch_count(int reset) {
  return reset ? g_launches.exchange(0, std::memory_order_relaxed) : g_launches.load(std::memory_order_relaxed);
}

int xaxb_set_wait_limit_ms(xaxb_ctx* ctx, int local_ms, int peer_ms) {
  if (!ctx || local_ms < 0 || peer_ms < 0) {
    set_last_error("set_wait_limit_ms: null context or negative limit");
    return XAXB_BAD_ARGUMENT;
  }
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  unsigned long long limits[2] = {local_ms ? (unsigned long long)local_ms * 1000000ull : kDefaultWaitLimitNs,
                                  peer_ms ? (unsigned long long)peer_ms * 1000000ull : kDefaultPeerWaitLimitNs};
  cudaError_t e = cudaSetDevice(c->device);
  // plain cudaMemcpy: ordered after all work already issued to the device, done when it returns
  if (e == cudaSuccess)
    e = cudaMemcpy(reinterpret_cast<unsigned char*>(c->d_status) + 8, limits, sizeof(limits), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    set_last_error("set_wait_limit_ms: %s", cudaGetErrorString(e));
    return XAXB_LAUNCH_FAILED;
  }
  return XAXB_OK;
}

}  // extern "C"
