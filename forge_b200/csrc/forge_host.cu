// Host-side helpers of the C ABI: error strings, device info cache, tensor-map encoding, status.
#include "forge_host.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

namespace forge {

static thread_local char g_err[512] = "no error";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

const char* last_error() { return g_err; }

static constexpr int kMaxDevices = 64;
static DeviceInfo g_info[kMaxDevices];
static bool g_info_valid[kMaxDevices];
static std::mutex g_info_mutex;

const DeviceInfo* current_device_info() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(FORGE_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_info_mutex);
  if (!g_info_valid[dev]) {
    DeviceInfo di;
    di.device = dev;
    if (cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&di.cc_minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
      fail(FORGE_ERR_CUDA, "cudaDeviceGetAttribute failed on device %d", dev);
      return nullptr;
    }
    g_info[dev] = di;
    g_info_valid[dev] = true;
  }
  return &g_info[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, bool is_float_type,
                   int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
                   int swizzle_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(FORGE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMapDataType dt;
  if (elem_bytes == 1) dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  else if (elem_bytes == 2) dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  else if (elem_bytes == 4) dt = is_float_type ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  else return fail(FORGE_ERR_INVALID_ARG, "tensor map: element size %d", elem_bytes);
  if (!aligned16(base)) return fail(FORGE_ERR_ALIGNMENT, "tensor base %p is not 16-byte aligned", base);
  if ((ld * elem_bytes) % 16 != 0)
    return fail(FORGE_ERR_ALIGNMENT, "row pitch of %lld bytes is not a multiple of 16",
                static_cast<long long>(ld * elem_bytes));
  if (rows <= 0 || cols <= 0 || ld < cols)
    return fail(FORGE_ERR_INVALID_ARG, "tensor map: rows=%lld cols=%lld ld=%lld", (long long)rows,
                (long long)cols, (long long)ld);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                      : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // a thread that has made no runtime call yet (e.g. an autograd worker) has no context bound:
    // bind the primary context of the current device and try once more
    cudaFree(nullptr);
    r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS)
    return fail(FORGE_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld)",
                static_cast<int>(r), (long long)rows, (long long)cols, (long long)ld);
  return FORGE_OK;
}

Hyper make_hyper(const ForgeHyper& h) {
  Hyper o;
  o.lr = static_cast<float>(h.lr);
  o.beta1 = static_cast<float>(h.beta1);
  o.beta2 = static_cast<float>(h.beta2);
  o.eps = static_cast<float>(h.eps);
  o.weight_decay = static_cast<float>(h.weight_decay);
  const double step = static_cast<double>(h.step > 0 ? h.step : 1);
  o.bc1 = static_cast<float>(1.0 - pow(h.beta1, step));
  o.bc2 = static_cast<float>(1.0 - pow(h.beta2, step));
  // 1 - beta and 1 - lr*wd in double first, then narrowed (the reference's PyTorch path passes them
  // as Python doubles: tests/test_correctness.py:43-44,52)
  o.one_m_beta1 = static_cast<float>(1.0 - h.beta1);
  o.one_m_beta2 = static_cast<float>(1.0 - h.beta2);
  o.decay = static_cast<float>(1.0 - h.lr * h.weight_decay);
  o.lr_over_bc1 = static_cast<float>(static_cast<double>(o.lr) / static_cast<double>(o.bc1));
  o.inv_bc2 = static_cast<float>(1.0 / static_cast<double>(o.bc2));
  o.momentum = static_cast<float>(h.momentum);
  o.nesterov = h.nesterov;
  return o;
}

}  // namespace forge

namespace forge {
const char* last_error();
}

extern "C" {

const char* forge_last_error_string(void) { return forge::last_error(); }

int forge_abi_version(void) { return FORGE_ABI_VERSION; }

int forge_read_status(int32_t* status, int32_t* code_out, void* cuda_stream) {
  if (status == nullptr || code_out == nullptr)
    return forge::fail(FORGE_ERR_INVALID_ARG, "forge_read_status: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return forge::fail(FORGE_ERR_CUDA, "forge_read_status: %s", cudaGetErrorString(e));
  *code_out = host;
  if (host != 0) {
    cudaMemsetAsync(status, 0, sizeof(int32_t), s);
    cudaStreamSynchronize(s);
    return forge::fail(FORGE_ERR_TIMEOUT, "a kernel abandoned a bounded wait (device code %d)", host);
  }
  return FORGE_OK;
}

int forge_state_bytes(int32_t optimizer, int32_t mode, int64_t V, int64_t H, int32_t qblock,
                      size_t* moment_bytes_each, size_t* scale_bytes_each, int32_t* num_moments) {
  if (V < 0 || H < 0 || moment_bytes_each == nullptr || scale_bytes_each == nullptr || num_moments == nullptr)
    return forge::fail(FORGE_ERR_INVALID_ARG, "forge_state_bytes: bad argument");
  int nm;
  switch (optimizer) {
    case FORGE_OPT_ADAMW: nm = 2; break;
    case FORGE_OPT_SGD: nm = 0; break;
    case FORGE_OPT_SGDM:
    case FORGE_OPT_LION: nm = 1; break;
    default: return forge::fail(FORGE_ERR_INVALID_ARG, "unknown optimizer %d", optimizer);
  }
  size_t es = 0, sc = 0;
  switch (mode) {
    case FORGE_ST_NONE: es = 0; break;
    case FORGE_ST_F32: es = 4; break;
    case FORGE_ST_BF16: es = 2; break;
    case FORGE_ST_INT8:
    case FORGE_ST_FP8_BLOCK:
      if (qblock <= 0 || H % qblock != 0)
        return forge::fail(FORGE_ERR_SHAPE, "H (%lld) must be divisible by qblock (%d)", (long long)H, qblock);
      es = 1;
      sc = static_cast<size_t>(V) * static_cast<size_t>(H / qblock) * sizeof(float);
      break;
    case FORGE_ST_FP8_TENSOR: es = 1; sc = sizeof(float); break;
    default: return forge::fail(FORGE_ERR_INVALID_ARG, "unknown state mode %d", mode);
  }
  if (nm == 0) { es = 0; sc = 0; }
  *num_moments = nm;
  *moment_bytes_each = es * static_cast<size_t>(V) * static_cast<size_t>(H);
  *scale_bytes_each = sc;
  return FORGE_OK;
}

}  // extern "C"
