// Optimizer-only update on a gradient that already exists in memory, and the fp8 delayed-scaling
// bookkeeping.  Same per-element arithmetic as the fused epilogue (forge_update.cuh), so feeding
// this kernel the fp32 gradient reproduces the fused kernel's W / moments / codes bit for bit.
//
// Layout of the work: one thread owns 16 consecutive columns of one row (128-bit loads and stores
// for every element type); four neighbouring lanes own one 64-column quantisation block and agree
// on its absmax with two shuffles.
#include <algorithm>

#include "forge_host.h"

namespace forge {

struct OptimParams {
  const void* grad;
  void* W;
  void* m;
  void* v;
  float* m_scale;
  float* v_scale;
  float* m_absmax;
  float* v_absmax;
  int64_t V, H;
  int64_t ld_grad, ld_w, ld_state, ld_scale;
  Hyper hyper;
};

template <int ES>
__device__ __forceinline__ void load16(const void* base, int64_t elem_off, float (&out)[16]) {
  if constexpr (ES == 4) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 q = p[i];
      out[4 * i + 0] = q.x; out[4 * i + 1] = q.y; out[4 * i + 2] = q.z; out[4 * i + 3] = q.w;
    }
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 q = p[i];
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        out[8 * i + 2 * k + 0] = __uint_as_float(u[k] << 16);
        out[8 * i + 2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u);
      }
    }
  }
}

template <int ES>
__device__ __forceinline__ void store16(void* base, int64_t elem_off, const float (&in)[16]) {
  if constexpr (ES == 4) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + elem_off);
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = make_float4(in[4 * i + 0], in[4 * i + 1], in[4 * i + 2], in[4 * i + 3]);
  } else {
    uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + elem_off);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        u[k] = float_to_bf16_bits(in[8 * i + 2 * k + 0]) | (float_to_bf16_bits(in[8 * i + 2 * k + 1]) << 16);
      p[i] = make_uint4(u[0], u[1], u[2], u[3]);
    }
  }
}

template <int G_DT, int W_DT, int ST, int OPT>
__global__ void __launch_bounds__(256) forge_optim_kernel(const OptimParams p) {
  constexpr int GES = (G_DT == DT_BF16) ? 2 : 4;
  constexpr int WES = (W_DT == DT_BF16) ? 2 : 4;
  constexpr int SES = (ST == ST_F32) ? 4 : 2;
  const Hyper hy = p.hyper;
  const int64_t groups_per_row = p.H / 16;
  const int64_t total = p.V * groups_per_row;
  // whole warps stay in the loop together (the block absmax uses warp shuffles): pad to 32
  const int64_t total_pad = (total + 31) & ~static_cast<int64_t>(31);
  float s_m_t = 1.0f, s_v_t = 1.0f, inv_m_t = 1.0f, inv_v_t = 1.0f, amax_m_t = 0.0f, amax_v_t = 0.0f;
  if constexpr (ST == ST_FP8_TENSOR) {
    s_m_t = *p.m_scale;
    s_v_t = *p.v_scale;
    inv_m_t = f_div(1.0f, s_m_t);
    inv_v_t = f_div(1.0f, s_v_t);
  }
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total_pad;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const bool live = idx < total;
    const int64_t row = live ? idx / groups_per_row : 0;
    const int64_t col = live ? (idx % groups_per_row) * 16 : 0;
    float g[16], w[16];
    if (live) {
      load16<GES>(p.grad, row * p.ld_grad + col, g);
      load16<WES>(p.W, row * p.ld_w + col, w);
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k) { g[k] = 0.0f; w[k] = 0.0f; }
    }
    if constexpr (OPT == OPT_SGD) {
#pragma unroll
      for (int k = 0; k < 16; ++k) w[k] = sgd_update(w[k], g[k], hy);
      if (live) store16<WES>(p.W, row * p.ld_w + col, w);
    } else if constexpr (OPT == OPT_SGDM || OPT == OPT_LION) {
      float m[16];
      if (live) load16<SES>(p.m, row * p.ld_state + col, m);
#pragma unroll
      for (int k = 0; k < 16; ++k)
        w[k] = (OPT == OPT_SGDM) ? sgdm_update(w[k], g[k], m[k], hy) : lion_update(w[k], g[k], m[k], hy);
      if (live) {
        store16<WES>(p.W, row * p.ld_w + col, w);
        store16<SES>(p.m, row * p.ld_state + col, m);
      }
    } else if constexpr (ST == ST_F32 || ST == ST_BF16) {
      float m[16], v[16];
      if (live) {
        load16<SES>(p.m, row * p.ld_state + col, m);
        load16<SES>(p.v, row * p.ld_state + col, v);
#pragma unroll
        for (int k = 0; k < 16; k += 2) {
          float2 m2 = make_float2(m[k], m[k + 1]), v2 = make_float2(v[k], v[k + 1]);
          const float2 w2 = adamw_update2(make_float2(w[k], w[k + 1]), make_float2(g[k], g[k + 1]), m2, v2, hy);
          w[k] = w2.x; w[k + 1] = w2.y;
          m[k] = m2.x; m[k + 1] = m2.y;
          v[k] = v2.x; v[k + 1] = v2.y;
        }
        store16<WES>(p.W, row * p.ld_w + col, w);
        store16<SES>(p.m, row * p.ld_state + col, m);
        store16<SES>(p.v, row * p.ld_state + col, v);
      }
    } else {
      // one-byte codes
      uint32_t mq[4] = {0, 0, 0, 0}, vq[4] = {0, 0, 0, 0};
      float sm_old = 1.0f, sv_old = 1.0f;
      if (live) {
        const uint4 a = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.m) + row * p.ld_state + col);
        const uint4 b = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.v) + row * p.ld_state + col);
        mq[0] = a.x; mq[1] = a.y; mq[2] = a.z; mq[3] = a.w;
        vq[0] = b.x; vq[1] = b.y; vq[2] = b.z; vq[3] = b.w;
        if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
          sm_old = p.m_scale[row * p.ld_scale + col / 64];
          sv_old = p.v_scale[row * p.ld_scale + col / 64];
        }
      }
      float m[16], v[16];
      float am = 0.0f, av = 0.0f;
      if constexpr (ST == ST_INT8) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { mq[j] ^= 0x80808080u; vq[j] ^= 0x80808080u; }
      }
#pragma unroll
      for (int k = 0; k < 16; k += 2) {
        float2 m2, v2;
        if constexpr (ST == ST_INT8) {
          m2 = fmul2(int8x2_to_float(mq[k >> 2], k & 3), make_float2(sm_old, sm_old));
          v2 = fmul2(int8x2_to_float(vq[k >> 2], k & 3), make_float2(sv_old, sv_old));
          v2.x = fmaxf(v2.x, 1e-8f);
          v2.y = fmaxf(v2.y, 1e-8f);
        } else if constexpr (ST == ST_FP8_BLOCK) {
          e4m3x2_to_float(mq[k >> 2] >> (8 * (k & 3)), m2.x, m2.y);
          e4m3x2_to_float(vq[k >> 2] >> (8 * (k & 3)), v2.x, v2.y);
          m2 = fmul2(m2, make_float2(sm_old, sm_old));
          v2 = fmul2(v2, make_float2(sv_old, sv_old));
          v2.x = fmaxf(v2.x, 1e-8f);
          v2.y = fmaxf(v2.y, 1e-8f);
        } else {
          e4m3x2_to_float(mq[k >> 2] >> (8 * (k & 3)), m2.x, m2.y);
          e5m2x2_to_float(vq[k >> 2] >> (8 * (k & 3)), v2.x, v2.y);
          m2 = fmul2(m2, make_float2(s_m_t, s_m_t));
          v2 = fmul2(v2, make_float2(s_v_t, s_v_t));
        }
        const float2 w2 = adamw_update2(make_float2(w[k], w[k + 1]), make_float2(g[k], g[k + 1]), m2, v2, hy);
        w[k] = w2.x; w[k + 1] = w2.y;
        m[k] = m2.x; m[k + 1] = m2.y;
        v[k] = v2.x; v[k + 1] = v2.y;
        am = fmaxf(am, fmaxf(fabsf(m2.x), fabsf(m2.y)));
        av = fmaxf(av, fmaxf(fabsf(v2.x), fabsf(v2.y)));
      }
      uint32_t mo[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
      if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
        // the four lanes of a 64-column block agree on its absmax
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
        av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 1));
        av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 2));
        const float sm_new = (ST == ST_INT8) ? int8_scale(am) : fp8blk_scale(am);
        const float sv_new = (ST == ST_INT8) ? int8_scale(av) : fp8blk_scale(av);
          const float rsm = f_rcp(sm_new), rsv = f_rcp(sv_new);
        const float2 nsm2 = make_float2(-sm_new, -sm_new), nsv2 = make_float2(-sv_new, -sv_new);
        const float2 rsm2 = make_float2(rsm, rsm), rsv2 = make_float2(rsv, rsv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = 4 * j;
          const float2 qm01 = div2_by_rcp(make_float2(m[k], m[k + 1]), nsm2, rsm2);
          const float2 qm23 = div2_by_rcp(make_float2(m[k + 2], m[k + 3]), nsm2, rsm2);
          const float2 qv01 = div2_by_rcp(make_float2(v[k], v[k + 1]), nsv2, rsv2);
          const float2 qv23 = div2_by_rcp(make_float2(v[k + 2], v[k + 3]), nsv2, rsv2);
          if constexpr (ST == ST_INT8) {
            mo[j] = int8x4_pack(int8x2_round(qm01), int8x2_round(qm23));
            vo[j] = int8x4_pack(int8x2_round(qv01), int8x2_round(qv23));
          } else {
            mo[j] = e4m3x2_code_bits(qm01.x, qm01.y) | (e4m3x2_code_bits(qm23.x, qm23.y) << 16);
            vo[j] = e4m3x2_code_bits(qv01.x, qv01.y) | (e4m3x2_code_bits(qv23.x, qv23.y) << 16);
          }
        }
        if (live && (col % 64) == 0) {
          p.m_scale[row * p.ld_scale + col / 64] = sm_new;
          p.v_scale[row * p.ld_scale + col / 64] = sv_new;
        }
      } else {
        amax_m_t = fmaxf(amax_m_t, am);
        amax_v_t = fmaxf(amax_v_t, av);
#pragma unroll
        for (int k = 0; k < 16; k += 2) {
          const float2 mc = fmul2(make_float2(m[k], m[k + 1]), make_float2(inv_m_t, inv_m_t));
          const float2 vc = fmul2(make_float2(v[k], v[k + 1]), make_float2(inv_v_t, inv_v_t));
          mo[k >> 2] |= e4m3x2_code_bits(mc.x, mc.y) << (8 * (k & 3));
          vo[k >> 2] |= e5m2x2_code_bits(vc.x, vc.y) << (8 * (k & 3));
        }
      }
      if (live) {
        store16<WES>(p.W, row * p.ld_w + col, w);
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.m) + row * p.ld_state + col) = make_uint4(mo[0], mo[1], mo[2], mo[3]);
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.v) + row * p.ld_state + col) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
      }
    }
  }
  if constexpr (ST == ST_FP8_TENSOR) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      amax_m_t = fmaxf(amax_m_t, __shfl_xor_sync(0xffffffffu, amax_m_t, o));
      amax_v_t = fmaxf(amax_v_t, __shfl_xor_sync(0xffffffffu, amax_v_t, o));
    }
    if ((threadIdx.x & 31) == 0) {
      atomicMax(reinterpret_cast<unsigned int*>(p.m_absmax), __float_as_uint(amax_m_t));
      atomicMax(reinterpret_cast<unsigned int*>(p.v_absmax), __float_as_uint(amax_v_t));
    }
  }
}

// scale <- clamp(absmax_next, 1e-8) / MAX, at most twice the previous scale; absmax_next <- 0
__global__ void fp8_prestep_kernel(float* m_scale, float* v_scale, float* m_amax, float* v_amax) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float mn = f_div(fmaxf(*m_amax, 1e-8f), 448.0f);
    float vn = f_div(fmaxf(*v_amax, 1e-8f), 57344.0f);
    const float ms = *m_scale, vs = *v_scale;
    if (ms > 0.0f) mn = fminf(mn, f_mul(ms, 2.0f));
    if (vs > 0.0f) vn = fminf(vn, f_mul(vs, 2.0f));
    *m_scale = mn;
    *v_scale = vn;
    *m_amax = 0.0f;
    *v_amax = 0.0f;
  }
}

template <int G_DT, int W_DT, int ST, int OPT>
static int launch_optim(const OptimParams& p, int sm_count, cudaStream_t stream) {
  const int64_t total = p.V * (p.H / 16);
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  blocks = std::max<int64_t>(1, std::min<int64_t>(blocks, static_cast<int64_t>(sm_count) * 8));
  forge_optim_kernel<G_DT, W_DT, ST, OPT><<<static_cast<int>(blocks), threads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "optimizer kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

template <int G_DT, int W_DT>
static int dispatch_optim(int opt, int st, const OptimParams& p, int sm_count, cudaStream_t s) {
#define FORGE_CASE(OPT_, ST_) \
  if (opt == OPT_ && st == ST_) return launch_optim<G_DT, W_DT, ST_, OPT_>(p, sm_count, s);
  FORGE_CASE(OPT_ADAMW, ST_BF16)
  FORGE_CASE(OPT_ADAMW, ST_F32)
  FORGE_CASE(OPT_ADAMW, ST_INT8)
  FORGE_CASE(OPT_ADAMW, ST_FP8_BLOCK)
  FORGE_CASE(OPT_ADAMW, ST_FP8_TENSOR)
  FORGE_CASE(OPT_SGD, ST_NONE)
  FORGE_CASE(OPT_SGDM, ST_BF16)
  FORGE_CASE(OPT_SGDM, ST_F32)
  FORGE_CASE(OPT_LION, ST_BF16)
  FORGE_CASE(OPT_LION, ST_F32)
#undef FORGE_CASE
  return fail(FORGE_ERR_UNSUPPORTED, "optimizer %d with state mode %d is not built", opt, st);
}

}  // namespace forge

using namespace forge;

extern "C" int forge_optimizer_update(const ForgeOptimArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_optimizer_update: args is NULL");
  const ForgeOptimArgs& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (a.V < 0 || a.H < 0) return fail(FORGE_ERR_INVALID_ARG, "negative dimension");
  if (a.V == 0 || a.H == 0) return FORGE_OK;
  if (a.grad == nullptr || a.W == nullptr) return fail(FORGE_ERR_INVALID_ARG, "grad or W is NULL");
  if (a.w_dtype != FORGE_DT_BF16 && a.w_dtype != FORGE_DT_F32) return fail(FORGE_ERR_INVALID_ARG, "unknown W dtype %d", a.w_dtype);
  if (a.grad_dtype != FORGE_DT_BF16 && a.grad_dtype != FORGE_DT_F32) return fail(FORGE_ERR_INVALID_ARG, "unknown grad dtype %d", a.grad_dtype);
  const int opt = a.optimizer;
  int st = a.state.mode;
  if (opt < FORGE_OPT_ADAMW || opt > FORGE_OPT_LION) return fail(FORGE_ERR_INVALID_ARG, "unknown optimizer %d", opt);
  if (opt == FORGE_OPT_SGD) st = FORGE_ST_NONE;
  if (opt != FORGE_OPT_SGD && (st < FORGE_ST_F32 || st > FORGE_ST_FP8_TENSOR)) return fail(FORGE_ERR_INVALID_ARG, "unknown state mode %d", st);
  if (a.hyper.step < 1 && opt == FORGE_OPT_ADAMW) return fail(FORGE_ERR_INVALID_ARG, "step must be >= 1 (got %d)", a.hyper.step);
  const int nm = opt == FORGE_OPT_ADAMW ? 2 : (opt == FORGE_OPT_SGD ? 0 : 1);
  if (nm > 0 && a.state.m == nullptr) return fail(FORGE_ERR_INVALID_ARG, "first moment buffer is NULL");
  if (nm > 1 && a.state.v == nullptr) return fail(FORGE_ERR_INVALID_ARG, "second moment buffer is NULL");
  const int ges = a.grad_dtype == FORGE_DT_BF16 ? 2 : 4;
  const int wes = a.w_dtype == FORGE_DT_BF16 ? 2 : 4;
  const int ses = st == FORGE_ST_F32 ? 4 : (st == FORGE_ST_BF16 ? 2 : (st == FORGE_ST_NONE ? 0 : 1));
  if (a.H % 16 != 0) return fail(FORGE_ERR_SHAPE, "H (%lld) must be a multiple of 16", (long long)a.H);
  if (!aligned16(a.grad) || !aligned16(a.W) || (nm > 0 && !aligned16(a.state.m)) || (nm > 1 && !aligned16(a.state.v)))
    return fail(FORGE_ERR_ALIGNMENT, "grad, W and the moments must be 16-byte aligned");
  if ((a.ld_grad * ges) % 16 != 0 || (a.ld_w * wes) % 16 != 0 || (nm > 0 && (a.state.ld_state * ses) % 16 != 0))
    return fail(FORGE_ERR_ALIGNMENT, "row pitches must be multiples of 16 bytes");
  if (st == FORGE_ST_INT8 || st == FORGE_ST_FP8_BLOCK) {
    if (a.state.qblock != 64) return fail(FORGE_ERR_SHAPE, "qblock must be 64 (got %d)", a.state.qblock);
    if (a.H % 64 != 0) return fail(FORGE_ERR_SHAPE, "H (%lld) must be divisible by qblock (64)", (long long)a.H);
    if (a.state.m_scale == nullptr || a.state.v_scale == nullptr) return fail(FORGE_ERR_INVALID_ARG, "scale arrays are NULL");
  }
  if (st == FORGE_ST_FP8_TENSOR &&
      (a.state.m_scale == nullptr || a.state.v_scale == nullptr || a.state.m_absmax_next == nullptr || a.state.v_absmax_next == nullptr))
    return fail(FORGE_ERR_INVALID_ARG, "fp8 per-tensor scale / absmax pointers are NULL");
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;

  OptimParams p;
  p.grad = a.grad; p.W = a.W; p.m = a.state.m; p.v = a.state.v;
  p.m_scale = a.state.m_scale; p.v_scale = a.state.v_scale;
  p.m_absmax = a.state.m_absmax_next; p.v_absmax = a.state.v_absmax_next;
  p.V = a.V; p.H = a.H; p.ld_grad = a.ld_grad; p.ld_w = a.ld_w;
  p.ld_state = a.state.ld_state; p.ld_scale = a.state.ld_scale;
  p.hyper = make_hyper(a.hyper);
  if (a.grad_dtype == FORGE_DT_F32) {
    if (a.w_dtype == FORGE_DT_BF16) return dispatch_optim<DT_F32, DT_BF16>(opt, st, p, di->sm_count, stream);
    return dispatch_optim<DT_F32, DT_F32>(opt, st, p, di->sm_count, stream);
  }
  if (a.w_dtype == FORGE_DT_BF16) return dispatch_optim<DT_BF16, DT_BF16>(opt, st, p, di->sm_count, stream);
  return dispatch_optim<DT_BF16, DT_F32>(opt, st, p, di->sm_count, stream);
}

extern "C" int forge_fp8_prestep(float* m_scale, float* v_scale, float* m_absmax_next, float* v_absmax_next,
                                 void* cuda_stream) {
  if (m_scale == nullptr || v_scale == nullptr || m_absmax_next == nullptr || v_absmax_next == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_fp8_prestep: null pointer");
  fp8_prestep_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(m_scale, v_scale, m_absmax_next, v_absmax_next);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "fp8 prestep launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}
