// RMSNorm forward (recompute) and backward for the linears that fold their preceding norm: the
// normalised activation is not kept between forward and backward but recomputed right before the
// fused weight-gradient update that consumes it.  Arithmetic of the reference's helpers
// (src/fused_grad_optimizer/fused_rmsnorm_linear.py:32-62):
//   forward   y = bf16( gamma * (x * rsqrt(mean(x^2) + eps)) )                      all in fp32
//   backward  dx = g gamma rrms - x (sum_h g gamma x) rrms^3 / H ;  dgamma = sum_rows g x rrms
// HBM-bound row kernels: one CTA works on a few rows, 16-byte accesses, the row is read once into
// registers.  dgamma is reduced in two fixed-order stages (per-CTA partial sums in caller scratch,
// then one pass over them), so the result is bit-reproducible from run to run.
#include <cuda_bf16.h>

#include <algorithm>

#include "forge_host.h"

namespace forge {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_H = NORM_THREADS * 8 * 8;   // eight 16-byte pieces per thread: H <= 16384

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                 // `red` may still be read from the previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) t += red[i];   // same order in every thread
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u[i]) : "f"(f[2 * i + 1]), "f"(f[2 * i]));
  return make_uint4(u[0], u[1], u[2], u[3]);
}

// PIECES = 16-byte pieces of a row per thread (H <= PIECES * 8 * NORM_THREADS)
template <int PIECES>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ y,
                   int rows, int H, long long ld_x, long long ld_y, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  const int npieces = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * ld_x);
    uint4 raw[PIECES];
    float ss = 0.0f;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int i = threadIdx.x + p * NORM_THREADS;
      if (i < npieces) {
        raw[p] = xr[i];
        float f[8];
        unpack8(raw[p], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
      }
    }
    const float rrms = rsqrtf(block_sum(ss, red) / static_cast<float>(H) + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + row * ld_y);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int i = threadIdx.x + p * NORM_THREADS;
      if (i < npieces) {
        float f[8], g[8];
        unpack8(raw[p], f);
        unpack8(reinterpret_cast<const uint4*>(gamma)[i], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = g[k] * (f[k] * rrms);
        yr[i] = pack8(f);
      }
    }
  }
}

// One CTA handles rows blockIdx.x, blockIdx.x + gridDim.x, ...; its column sums of g * x * rrms go to
// partial[blockIdx.x][H] (fp32), summed over the CTAs by rmsnorm_dgamma_kernel in a fixed order.
template <int PIECES>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ gy, __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                   int rows, int H, long long ld_x, long long ld_gy, long long ld_dx, float eps) {
  __shared__ float red[NORM_THREADS / 32];
  const int npieces = H / 8;
  float acc[PIECES][8];
#pragma unroll
  for (int p = 0; p < PIECES; ++p)
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[p][k] = 0.0f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * ld_x);
    const uint4* gr = reinterpret_cast<const uint4*>(gy + row * ld_gy);
    uint4 rx[PIECES], rg[PIECES];
    float ss = 0.0f, sgx = 0.0f;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int i = threadIdx.x + p * NORM_THREADS;
      if (i < npieces) {
        rx[p] = xr[i];
        rg[p] = gr[i];
        float f[8], g[8], gm[8];
        unpack8(rx[p], f);
        unpack8(rg[p], g);
        unpack8(reinterpret_cast<const uint4*>(gamma)[i], gm);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          ss += f[k] * f[k];
          sgx += (g[k] * gm[k]) * f[k];
        }
      }
    }
    const float rrms = rsqrtf(block_sum(ss, red) / static_cast<float>(H) + eps);
    const float coef = block_sum(sgx, red) * rrms * rrms * rrms / static_cast<float>(H);
    uint4* dr = reinterpret_cast<uint4*>(dx + row * ld_dx);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int i = threadIdx.x + p * NORM_THREADS;
      if (i < npieces) {
        float f[8], g[8], gm[8], o[8];
        unpack8(rx[p], f);
        unpack8(rg[p], g);
        unpack8(reinterpret_cast<const uint4*>(gamma)[i], gm);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          o[k] = (g[k] * gm[k]) * rrms - f[k] * coef;
          acc[p][k] += g[k] * (f[k] * rrms);
        }
        dr[i] = pack8(o);
      }
    }
  }
  float* pr = partial + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) {
    const int i = threadIdx.x + p * NORM_THREADS;
    if (i < npieces) {
#pragma unroll
      for (int k = 0; k < 8; ++k) pr[i * 8 + k] = acc[p][k];
    }
  }
}

__global__ void rmsnorm_dgamma_kernel(const float* __restrict__ partial, int nparts, int H, float* __restrict__ dgamma_f32,
                                      __nv_bfloat16* __restrict__ dgamma_bf16, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.0f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<size_t>(p) * H + c];
  if (dgamma_f32 != nullptr) dgamma_f32[c] = accumulate ? dgamma_f32[c] + s : s;
  if (dgamma_bf16 != nullptr)
    dgamma_bf16[c] = __float2bfloat16_rn(accumulate ? __bfloat162float(dgamma_bf16[c]) + s : s);
}

static int norm_grid(int64_t rows, int sm_count) { return static_cast<int>(std::min<int64_t>(rows, 2 * sm_count)); }

static int check_norm_args(const void* x, int64_t rows, int64_t H, int64_t ld) {
  if (rows < 0 || H <= 0) return fail(FORGE_ERR_INVALID_ARG, "rmsnorm: bad shape %lld x %lld", (long long)rows, (long long)H);
  if (H % 8 != 0 || H > NORM_MAX_H) return fail(FORGE_ERR_SHAPE, "rmsnorm: H (%lld) must be a multiple of 8 and at most %d", (long long)H, NORM_MAX_H);
  if (x == nullptr || !aligned16(x) || (ld * 2) % 16 != 0) return fail(FORGE_ERR_ALIGNMENT, "rmsnorm: pointer or row pitch not 16-byte aligned");
  return FORGE_OK;
}

}  // namespace forge

using namespace forge;

extern "C" size_t forge_rmsnorm_backward_scratch_bytes(int64_t rows, int64_t H) {
  if (rows <= 0 || H <= 0) return 0;
  // one row of fp32 partial sums per CTA; the grid never exceeds two CTAs per SM of the largest part (148 SMs)
  return static_cast<size_t>(std::min<int64_t>(rows, 2 * 148)) * static_cast<size_t>(H) * sizeof(float);
}

extern "C" int forge_rmsnorm_forward(const void* x, const void* gamma, void* y, int64_t rows, int64_t H, int64_t ld_x,
                                     int64_t ld_y, double eps, void* cuda_stream) {
  int rc;
  if ((rc = check_norm_args(x, rows, H, ld_x)) != FORGE_OK) return rc;
  if ((rc = check_norm_args(y, rows, H, ld_y)) != FORGE_OK) return rc;
  if (gamma == nullptr || !aligned16(gamma)) return fail(FORGE_ERR_ALIGNMENT, "rmsnorm: gamma is NULL or not 16-byte aligned");
  if (rows == 0) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const int grid = norm_grid(rows, di->sm_count);
  const int pieces = static_cast<int>((H / 8 + NORM_THREADS - 1) / NORM_THREADS);
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto gb = static_cast<const __nv_bfloat16*>(gamma);
  auto yb = static_cast<__nv_bfloat16*>(y);
  const float e = static_cast<float>(eps);
  if (pieces <= 2) rmsnorm_fwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(xb, gb, yb, (int)rows, (int)H, ld_x, ld_y, e);
  else if (pieces <= 4) rmsnorm_fwd_kernel<4><<<grid, NORM_THREADS, 0, s>>>(xb, gb, yb, (int)rows, (int)H, ld_x, ld_y, e);
  else rmsnorm_fwd_kernel<8><<<grid, NORM_THREADS, 0, s>>>(xb, gb, yb, (int)rows, (int)H, ld_x, ld_y, e);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(FORGE_ERR_CUDA, "rmsnorm forward launch: %s", cudaGetErrorString(err));
  return FORGE_OK;
}

extern "C" int forge_rmsnorm_backward(const void* x, const void* gamma, const void* grad_y, void* grad_x, void* grad_gamma,
                                      int32_t grad_gamma_dtype, int32_t accumulate, int64_t rows, int64_t H, int64_t ld_x,
                                      int64_t ld_gy, int64_t ld_gx, double eps, void* scratch, size_t scratch_bytes,
                                      void* cuda_stream) {
  int rc;
  if ((rc = check_norm_args(x, rows, H, ld_x)) != FORGE_OK) return rc;
  if ((rc = check_norm_args(grad_y, rows, H, ld_gy)) != FORGE_OK) return rc;
  if ((rc = check_norm_args(grad_x, rows, H, ld_gx)) != FORGE_OK) return rc;
  if (gamma == nullptr || !aligned16(gamma) || grad_gamma == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "rmsnorm backward: gamma / grad_gamma is NULL or misaligned");
  if (grad_gamma_dtype != FORGE_DT_BF16 && grad_gamma_dtype != FORGE_DT_F32)
    return fail(FORGE_ERR_INVALID_ARG, "rmsnorm backward: unknown grad_gamma dtype %d", grad_gamma_dtype);
  if (rows == 0) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  const int grid = norm_grid(rows, di->sm_count);
  const size_t need = static_cast<size_t>(grid) * static_cast<size_t>(H) * sizeof(float);
  if (scratch == nullptr || scratch_bytes < need || !aligned16(scratch))
    return fail(FORGE_ERR_SCRATCH, "rmsnorm backward needs %zu bytes of 16-byte aligned scratch (got %zu)", need, scratch_bytes);
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  const int pieces = static_cast<int>((H / 8 + NORM_THREADS - 1) / NORM_THREADS);
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto gb = static_cast<const __nv_bfloat16*>(gamma);
  auto gy = static_cast<const __nv_bfloat16*>(grad_y);
  auto gx = static_cast<__nv_bfloat16*>(grad_x);
  float* part = static_cast<float*>(scratch);
  const float e = static_cast<float>(eps);
  if (pieces <= 2) rmsnorm_bwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(xb, gb, gy, gx, part, (int)rows, (int)H, ld_x, ld_gy, ld_gx, e);
  else if (pieces <= 4) rmsnorm_bwd_kernel<4><<<grid, NORM_THREADS, 0, s>>>(xb, gb, gy, gx, part, (int)rows, (int)H, ld_x, ld_gy, ld_gx, e);
  else rmsnorm_bwd_kernel<8><<<grid, NORM_THREADS, 0, s>>>(xb, gb, gy, gx, part, (int)rows, (int)H, ld_x, ld_gy, ld_gx, e);
  rmsnorm_dgamma_kernel<<<static_cast<int>((H + 255) / 256), 256, 0, s>>>(
      part, grid, (int)H, grad_gamma_dtype == FORGE_DT_F32 ? static_cast<float*>(grad_gamma) : nullptr,
      grad_gamma_dtype == FORGE_DT_BF16 ? static_cast<__nv_bfloat16*>(grad_gamma) : nullptr, accumulate);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(FORGE_ERR_CUDA, "rmsnorm backward launch: %s", cudaGetErrorString(err));
  return FORGE_OK;
}
