// Fused weight-gradient + optimizer kernel for sm_100a.
//
//   dW[v,h] = sum_bt dY[bt,v] * X[bt,h]          (bf16 x bf16, fp32 accumulate in tensor memory)
//   (W, moments)[v,h] <- optimizer(W, moments, dW)   applied to the accumulator tile on chip
//
// No gradient tensor is written to global memory.  This replaces, for one launch per linear, the
// reference's fused kernels (src/fused_grad_optimizer/kernel.py:212-317 AdamW, :122-205 SGD,
// :324-478 int8 moments, kernel_fp8_state.py:204-295 fp8 moments).
//
// Structure: one persistent CTA per SM, 12 warps.
//   warp 0      TMA producer of the dY / X panels (both operands are M/N-major in memory: dY is
//               (BT,V) with V contiguous, X is (BT,H) with H contiguous; no transpose is made)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), frees it
//   warp 2      TMA producer of the W / moment sub-tiles (prefetched while the MMAs of the tile run)
//   warp 3      idle
//   warps 4-11  epilogue: two groups of four warps; group g handles the 64-column chunks g and g+2
//               of the 128 x 256 tile.  Each thread owns one accumulator row: tcgen05.ld, fp32
//               update against the staged W/moment rows in shared memory (in place), then one TMA
//               store per warp and tensor.
// Tensor memory holds two 128 x 256 fp32 accumulators, so the MMAs of tile i+1 overlap the
// epilogue of tile i.
#pragma once

#include "forge_ptx.cuh"
#include "forge_update.cuh"

namespace forge {

constexpr int TILE_M = 128;        // rows of W per tile (V direction)
constexpr int TILE_N = 256;        // columns of W per tile (H direction)
constexpr int CHUNK_N = 64;        // columns per epilogue chunk
constexpr int NUM_CHUNKS = TILE_N / CHUNK_N;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 384;
constexpr int EPI_WARP0 = 4;
constexpr int NUM_EPI_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BUDGET = 227 * 1024;

// error codes written to the status word
enum : int {
  ERR_WAIT_OP_EMPTY = 101,
  ERR_WAIT_OP_FULL = 102,
  ERR_WAIT_ST_EMPTY = 103,
  ERR_WAIT_ST_FULL = 104,
  ERR_WAIT_ACC_EMPTY = 105,
  ERR_WAIT_ACC_FULL = 106
};

template <int ES>
struct BoxGeom;  // geometry of one 128-row x 64-column chunk of a tensor with ES-byte elements
template <>
struct BoxGeom<2> {  // one box: 64 columns = 128 bytes per row, 128-byte swizzle
  static constexpr int kBoxes = 1, kBoxCols = 64, kPitch = 128, kBoxBytes = 128 * 128;
};
template <>
struct BoxGeom<4> {  // two boxes of 32 columns = 128 bytes per row each, 128-byte swizzle
  static constexpr int kBoxes = 2, kBoxCols = 32, kPitch = 128, kBoxBytes = 128 * 128;
};
template <>
struct BoxGeom<1> {  // one box: 64 columns = 64 bytes per row, 64-byte swizzle
  static constexpr int kBoxes = 1, kBoxCols = 64, kPitch = 64, kBoxBytes = 128 * 64;
};

template <int ES>
__host__ __device__ constexpr int chunk_bytes() {
  return 128 * CHUNK_N * ES;
}

__host__ __device__ constexpr int num_moments(int opt) {
  return opt == OPT_ADAMW ? 2 : (opt == OPT_SGD ? 0 : 1);
}
__host__ __device__ constexpr int state_elem_size(int st) {
  return st == ST_F32 ? 4 : (st == ST_BF16 ? 2 : (st == ST_NONE ? 0 : 1));
}

// byte offset of the 16-byte piece `j` of row `r` inside a chunk buffer
template <int ES>
__device__ __forceinline__ uint32_t piece_off(int r, int j) {
  if constexpr (ES == 2) {
    return r * 128 + ((j ^ (r & 7)) << 4);
  } else if constexpr (ES == 4) {
    return (j >> 3) * BoxGeom<4>::kBoxBytes + r * 128 + (((j & 7) ^ (r & 7)) << 4);
  } else {
    return r * 64 + ((j ^ ((r >> 1) & 3)) << 4);
  }
}

// ---- 16-element row-group loads / stores between shared memory and fp32 registers -------------
template <int ES>
__device__ __forceinline__ void ld16_float(const uint8_t* buf, int r, int g, float (&out)[16]) {
  if constexpr (ES == 4) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float4 q = *reinterpret_cast<const float4*>(buf + piece_off<4>(r, 4 * g + p));
      out[4 * p + 0] = q.x; out[4 * p + 1] = q.y; out[4 * p + 2] = q.z; out[4 * p + 3] = q.w;
    }
  } else {
    static_assert(ES == 2, "float/bf16 only");
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const uint4 q = *reinterpret_cast<const uint4*>(buf + piece_off<2>(r, 2 * g + p));
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[8 * p + 2 * i + 0] = __uint_as_float(u[i] << 16);
        out[8 * p + 2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
      }
    }
  }
}

template <int ES>
__device__ __forceinline__ void st16_float(uint8_t* buf, int r, int g, const float (&in)[16]) {
  if constexpr (ES == 4) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      *reinterpret_cast<float4*>(buf + piece_off<4>(r, 4 * g + p)) =
          make_float4(in[4 * p + 0], in[4 * p + 1], in[4 * p + 2], in[4 * p + 3]);
    }
  } else {
    static_assert(ES == 2, "float/bf16 only");
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      uint32_t u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        u[i] = float_to_bf16_bits(in[8 * p + 2 * i + 0]) |
               (float_to_bf16_bits(in[8 * p + 2 * i + 1]) << 16);
      }
      *reinterpret_cast<uint4*>(buf + piece_off<2>(r, 2 * g + p)) = make_uint4(u[0], u[1], u[2], u[3]);
    }
  }
}

__device__ __forceinline__ void ld16_bytes(const uint8_t* buf, int r, int g, uint32_t (&w)[4]) {
  const uint4 q = *reinterpret_cast<const uint4*>(buf + piece_off<1>(r, g));
  w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
}
__device__ __forceinline__ void st16_bytes(uint8_t* buf, int r, int g, const uint32_t (&w)[4]) {
  *reinterpret_cast<uint4*>(buf + piece_off<1>(r, g)) = make_uint4(w[0], w[1], w[2], w[3]);
}

// kernel parameters ------------------------------------------------------------------------------
struct WgradParams {
  int BT, V, H;
  int num_kb;          // ceil(BT / BK)
  int tiles_m, tiles_n;
  Hyper hyper;
  float* m_scale;      // int8 / fp8-block: (V, H/64) row-major; fp8-tensor: one scalar
  float* v_scale;
  int ld_scale;        // row pitch of the scale arrays, in floats
  float* m_absmax;     // fp8-tensor: next-step absmax accumulators (atomic max)
  float* v_absmax;
  int* status;         // device status word: 0 = ok
};

template <int BK, int NSTAGE>
__host__ __device__ constexpr int op_stage_bytes() {
  return (TILE_M + TILE_N) * BK * 2;
}

template <int W_DT, int ST, int OPT>
struct WgradCfg {
  static constexpr int kWES = (W_DT == DT_BF16) ? 2 : 4;
  static constexpr int kNMom = num_moments(OPT);
  static constexpr int kSES = state_elem_size(ST);
  static constexpr int kWBytes = chunk_bytes<kWES>();
  static constexpr int kSBytes = (kNMom > 0) ? 128 * CHUNK_N * kSES : 0;
  static constexpr int kStageBytes = kWBytes + kNMom * kSBytes;
  static constexpr int kBK = 64;
  static constexpr int kOpStageBytes = (TILE_M + TILE_N) * kBK * 2;
  static constexpr int kCtrlBytes = 1024;
  // two operand stages when that still leaves room for two state stages, else fit what we can
  static constexpr int kNStage = 2;
  static constexpr int kRoom = SMEM_BUDGET - kCtrlBytes - 1024 - kNStage * kOpStageBytes;
  static constexpr int kNSS_raw = kRoom / kStageBytes;
  static constexpr int kNSS = kNSS_raw > 4 ? 4 : kNSS_raw;
  static constexpr int kSmemBytes = kCtrlBytes + 1024 + kNStage * kOpStageBytes + kNSS * kStageBytes;
  static_assert(kNSS >= 1, "state stage does not fit in shared memory");
};

struct alignas(8) CtrlBlock {
  uint64_t op_full[4];
  uint64_t op_empty[4];
  uint64_t st_full[4];
  uint64_t st_empty[4];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_word;
};

// ------------------------------------------------------------------------------------------------
template <int W_DT, int ST, int OPT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
forge_wgrad_kernel(const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_x,
                   const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_m,
                   const __grid_constant__ CUtensorMap tm_v, const WgradParams p) {
  using Cfg = WgradCfg<W_DT, ST, OPT>;
  constexpr int BK = Cfg::kBK;
  constexpr int NSTAGE = Cfg::kNStage;
  constexpr int NSS = Cfg::kNSS;
  constexpr int WES = Cfg::kWES;
  constexpr int SES = Cfg::kSES;
  constexpr int NMOM = Cfg::kNMom;
  constexpr int A_BYTES = TILE_M * BK * 2;
  constexpr int B_BYTES = TILE_N * BK * 2;
  constexpr int SLAB_BYTES = 64 * BK * 2;  // one 64-element M/N slab of a K panel

  extern __shared__ uint8_t smem_raw[];
  // control block first, then 1024-byte aligned data
  CtrlBlock* ctrl = reinterpret_cast<CtrlBlock*>(smem_raw);
  uint8_t* data = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + Cfg::kCtrlBytes + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* op_buf = data;                                   // NSTAGE x (A | B)
  uint8_t* st_buf = data + NSTAGE * Cfg::kOpStageBytes;     // NSS x (W | m | v)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_word = &ctrl->abort_word;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&ctrl->op_full[i], 1); mbar_init(&ctrl->op_empty[i], 1); }
    for (int i = 0; i < NSS; ++i) { mbar_init(&ctrl->st_full[i], 1); mbar_init(&ctrl->st_empty[i], 4); }
    for (int i = 0; i < 2; ++i) { mbar_init(&ctrl->acc_full[i], 1); mbar_init(&ctrl->acc_empty[i], NUM_EPI_WARPS); }
    ctrl->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tm_dy); prefetch_tmap(&tm_x); }
  if (warp == 2 && lane == 0) {
    prefetch_tmap(&tm_w);
    if (NMOM > 0) prefetch_tmap(&tm_m);
    if (NMOM > 1) prefetch_tmap(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------------ operand producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int row0 = (tile / p.tiles_n) * TILE_M;
        const int col0 = (tile % p.tiles_n) * TILE_N;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          if (!mbar_wait(&ctrl->op_empty[s], ph ^ 1, abort_word, ERR_WAIT_OP_EMPTY)) goto done;
          uint8_t* a = op_buf + s * Cfg::kOpStageBytes;
          uint8_t* b = a + A_BYTES;
          mbar_expect_tx(&ctrl->op_full[s], A_BYTES + B_BYTES);
#pragma unroll
          for (int i = 0; i < TILE_M / 64; ++i)
            tma_load_2d(a + i * SLAB_BYTES, &tm_dy, &ctrl->op_full[s], row0 + 64 * i, kb * BK, pol);
#pragma unroll
          for (int i = 0; i < TILE_N / 64; ++i)
            tma_load_2d(b + i * SLAB_BYTES, &tm_x, &ctrl->op_full[s], col0 + 64 * i, kb * BK, pol);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, TILE_N, true, true);
      uint32_t it = 0;
      uint32_t tile_it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_it) {
        const int buf = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&ctrl->acc_empty[buf], aph ^ 1, abort_word, ERR_WAIT_ACC_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * TILE_N;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          if (!mbar_wait(&ctrl->op_full[s], ph, abort_word, ERR_WAIT_OP_FULL)) goto done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(op_buf + s * Cfg::kOpStageBytes);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 rows = two 1024-byte swizzle atoms
            const uint64_t da = make_smem_desc_sw128(a_addr + k * (UMMA_K * 128), SLAB_BYTES, 1024);
            const uint64_t db = make_smem_desc_sw128(b_addr + k * (UMMA_K * 128), SLAB_BYTES, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&ctrl->op_empty[s]);
        }
        umma_commit(&ctrl->acc_full[buf]);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ state producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_first();
      uint32_t q = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        const int row0 = (tile / p.tiles_n) * TILE_M;
        const int col0 = (tile % p.tiles_n) * TILE_N;
        for (int c = 0; c < NUM_CHUNKS; ++c, ++q) {
          const int s = q % NSS;
          const uint32_t ph = (q / NSS) & 1;
          if (!mbar_wait(&ctrl->st_empty[s], ph ^ 1, abort_word, ERR_WAIT_ST_EMPTY)) goto done;
          uint8_t* wb = st_buf + s * Cfg::kStageBytes;
          mbar_expect_tx(&ctrl->st_full[s], Cfg::kStageBytes);
          const int cc = col0 + c * CHUNK_N;
#pragma unroll
          for (int rb = 0; rb < 4; ++rb) {
            const int rr = row0 + 32 * rb;
#pragma unroll
            for (int bx = 0; bx < BoxGeom<WES>::kBoxes; ++bx)
              tma_load_2d(wb + bx * BoxGeom<WES>::kBoxBytes + rb * 32 * BoxGeom<WES>::kPitch, &tm_w,
                          &ctrl->st_full[s], cc + bx * BoxGeom<WES>::kBoxCols, rr, pol);
            if constexpr (NMOM > 0) {
              uint8_t* mb = wb + Cfg::kWBytes;
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SES>::kBoxes; ++bx)
                tma_load_2d(mb + bx * BoxGeom<SES>::kBoxBytes + rb * 32 * BoxGeom<SES>::kPitch, &tm_m,
                            &ctrl->st_full[s], cc + bx * BoxGeom<SES>::kBoxCols, rr, pol);
            }
            if constexpr (NMOM > 1) {
              uint8_t* vb = wb + Cfg::kWBytes + Cfg::kSBytes;
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SES>::kBoxes; ++bx)
                tma_load_2d(vb + bx * BoxGeom<SES>::kBoxBytes + rb * 32 * BoxGeom<SES>::kPitch, &tm_v,
                            &ctrl->st_full[s], cc + bx * BoxGeom<SES>::kBoxCols, rr, pol);
            }
          }
        }
      }
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int wg = (warp - EPI_WARP0) >> 2;       // 0 or 1
    const int r = quarter * 32 + lane;            // row inside the tile
    const Hyper hy = p.hyper;
    const uint64_t pol = policy_evict_first();
    float s_m_t = 1.0f, s_v_t = 1.0f, inv_m_t = 1.0f, inv_v_t = 1.0f;
    float amax_m_t = 0.0f, amax_v_t = 0.0f;
    if constexpr (ST == ST_FP8_TENSOR) {
      s_m_t = *p.m_scale;
      s_v_t = *p.v_scale;
      inv_m_t = f_div(1.0f, s_m_t);
      inv_v_t = f_div(1.0f, s_v_t);
    }
    uint32_t tile_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tile_it) {
      const int row0 = (tile / p.tiles_n) * TILE_M;
      const int col0 = (tile % p.tiles_n) * TILE_N;
      const int buf = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const int grow = row0 + r;

      // per-(row, 64-column block) scales of this thread's two chunks
      float sc_m[2] = {1.0f, 1.0f}, sc_v[2] = {1.0f, 1.0f};
      if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int cb = (col0 >> 6) + wg + 2 * i;
          if (grow < p.V && cb * 64 < p.H) {
            sc_m[i] = __ldg(p.m_scale + static_cast<size_t>(grow) * p.ld_scale + cb);
            sc_v[i] = __ldg(p.v_scale + static_cast<size_t>(grow) * p.ld_scale + cb);
          }
        }
      }

      ok = mbar_wait(&ctrl->acc_full[buf], aph, abort_word, ERR_WAIT_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

#pragma unroll 1
      for (int i = 0; i < 2; ++i) {
        const int c = wg + 2 * i;
        const uint32_t q = tile_it * NUM_CHUNKS + c;
        const int s = q % NSS;
        const uint32_t ph = (q / NSS) & 1;

        // accumulator row: 64 fp32 columns of this chunk
        uint32_t acc[64];
        {
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(buf * TILE_N + c * CHUNK_N);
          tmem_ld_32x32(taddr, &acc[0]);
          tmem_ld_32x32(taddr + 32, &acc[32]);
        }
        ok = mbar_wait(&ctrl->st_full[s], ph, abort_word, ERR_WAIT_ST_FULL);
        ok = __all_sync(0xffffffffu, ok);
        tmem_ld_wait();
        if (!ok) break;
        if (p.num_kb == 0) {
#pragma unroll
          for (int k = 0; k < 64; ++k) acc[k] = 0u;
        }

        uint8_t* wb = st_buf + s * Cfg::kStageBytes;
        uint8_t* mb = wb + Cfg::kWBytes;
        uint8_t* vb = mb + Cfg::kSBytes;

        if constexpr (OPT == OPT_SGD) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[16];
            ld16_float<WES>(wb, r, g, w);
#pragma unroll
            for (int k = 0; k < 16; ++k) w[k] = sgd_update(w[k], __uint_as_float(acc[16 * g + k]), hy);
            st16_float<WES>(wb, r, g, w);
          }
        } else if constexpr (OPT == OPT_SGDM || OPT == OPT_LION) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[16], m[16];
            ld16_float<WES>(wb, r, g, w);
            ld16_float<SES>(mb, r, g, m);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float gr = __uint_as_float(acc[16 * g + k]);
              w[k] = (OPT == OPT_SGDM) ? sgdm_update(w[k], gr, m[k], hy) : lion_update(w[k], gr, m[k], hy);
            }
            st16_float<WES>(wb, r, g, w);
            st16_float<SES>(mb, r, g, m);
          }
        } else if constexpr (ST == ST_F32 || ST == ST_BF16) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[16], m[16], v[16];
            ld16_float<WES>(wb, r, g, w);
            ld16_float<SES>(mb, r, g, m);
            ld16_float<SES>(vb, r, g, v);
#pragma unroll
            for (int k = 0; k < 16; ++k)
              w[k] = adamw_update(w[k], __uint_as_float(acc[16 * g + k]), m[k], v[k], hy);
            st16_float<WES>(wb, r, g, w);
            st16_float<SES>(mb, r, g, m);
            st16_float<SES>(vb, r, g, v);
          }
        } else if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
          // pass 1: dequantise, update W, find the block absmax of the new moments
          const float sm_old = sc_m[i], sv_old = sc_v[i];
          float am = 0.0f, av = 0.0f;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[16];
            uint32_t mq[4], vq[4];
            ld16_float<WES>(wb, r, g, w);
            ld16_bytes(mb, r, g, mq);
            ld16_bytes(vb, r, g, vq);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t mbits = (mq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              const uint32_t vbits = (vq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              float m, v;
              if constexpr (ST == ST_INT8) {
                m = f_mul(static_cast<float>(static_cast<int>(static_cast<int8_t>(mbits))), sm_old);
                v = fmaxf(f_mul(static_cast<float>(static_cast<int>(static_cast<int8_t>(vbits))), sv_old), 1e-8f);
              } else {
                m = f_mul(e4m3_to_float(static_cast<uint8_t>(mbits)), sm_old);
                v = fmaxf(f_mul(e4m3_to_float(static_cast<uint8_t>(vbits)), sv_old), 1e-8f);
              }
              w[k] = adamw_update(w[k], __uint_as_float(acc[16 * g + k]), m, v, hy);
              am = fmaxf(am, fabsf(m));
              av = fmaxf(av, fabsf(v));
            }
            st16_float<WES>(wb, r, g, w);
          }
          const float sm_new = (ST == ST_INT8) ? int8_scale(am) : fp8blk_scale(am);
          const float sv_new = (ST == ST_INT8) ? int8_scale(av) : fp8blk_scale(av);
          // pass 2: recompute the new moments (same instruction sequence) and requantise
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t mq[4], vq[4], mo[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
            ld16_bytes(mb, r, g, mq);
            ld16_bytes(vb, r, g, vq);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t mbits = (mq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              const uint32_t vbits = (vq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              const float gr = __uint_as_float(acc[16 * g + k]);
              float m, v;
              if constexpr (ST == ST_INT8) {
                m = f_mul(static_cast<float>(static_cast<int>(static_cast<int8_t>(mbits))), sm_old);
                v = fmaxf(f_mul(static_cast<float>(static_cast<int>(static_cast<int8_t>(vbits))), sv_old), 1e-8f);
              } else {
                m = f_mul(e4m3_to_float(static_cast<uint8_t>(mbits)), sm_old);
                v = fmaxf(f_mul(e4m3_to_float(static_cast<uint8_t>(vbits)), sv_old), 1e-8f);
              }
              m = f_add(f_mul(hy.beta1, m), f_mul(hy.one_m_beta1, gr));
              v = f_add(f_mul(hy.beta2, v), f_mul(f_mul(hy.one_m_beta2, gr), gr));
              uint32_t mc, vc;
              if constexpr (ST == ST_INT8) {
                mc = static_cast<uint32_t>(int8_code(m, sm_new)) & 0xFFu;
                vc = static_cast<uint32_t>(int8_code(v, sv_new)) & 0xFFu;
              } else {
                mc = e4m3_code(f_div(m, sm_new));
                vc = e4m3_code(f_div(v, sv_new));
              }
              mo[k >> 2] |= mc << (8 * (k & 3));
              vo[k >> 2] |= vc << (8 * (k & 3));
            }
            st16_bytes(mb, r, g, mo);
            st16_bytes(vb, r, g, vo);
          }
          {
            const int cb = (col0 >> 6) + c;
            if (grow < p.V && cb * 64 < p.H) {
              p.m_scale[static_cast<size_t>(grow) * p.ld_scale + cb] = sm_new;
              p.v_scale[static_cast<size_t>(grow) * p.ld_scale + cb] = sv_new;
            }
          }
        } else {  // ST_FP8_TENSOR
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float w[16];
            uint32_t mq[4], vq[4], mo[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
            ld16_float<WES>(wb, r, g, w);
            ld16_bytes(mb, r, g, mq);
            ld16_bytes(vb, r, g, vq);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t mbits = (mq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              const uint32_t vbits = (vq[k >> 2] >> (8 * (k & 3))) & 0xFFu;
              float m = f_mul(e4m3_to_float(static_cast<uint8_t>(mbits)), s_m_t);
              float v = f_mul(e5m2_to_float(static_cast<uint8_t>(vbits)), s_v_t);
              w[k] = adamw_update(w[k], __uint_as_float(acc[16 * g + k]), m, v, hy);
              // rows / columns beyond the matrix hold zeros (zero-filled loads), so they never
              // raise the running maxima
              amax_m_t = fmaxf(amax_m_t, fabsf(m));
              amax_v_t = fmaxf(amax_v_t, fabsf(v));
              mo[k >> 2] |= static_cast<uint32_t>(e4m3_code(f_mul(m, inv_m_t))) << (8 * (k & 3));
              vo[k >> 2] |= static_cast<uint32_t>(e5m2_code(f_mul(v, inv_v_t))) << (8 * (k & 3));
            }
            st16_float<WES>(wb, r, g, w);
            st16_bytes(mb, r, g, mo);
            st16_bytes(vb, r, g, vo);
          }
        }

        // hand the updated rows of this warp to the TMA store engine
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int rr = row0 + quarter * 32;
          const int cc = col0 + c * CHUNK_N;
          if (rr < p.V && cc < p.H) {
#pragma unroll
            for (int bx = 0; bx < BoxGeom<WES>::kBoxes; ++bx)
              if (cc + bx * BoxGeom<WES>::kBoxCols < p.H)
                tma_store_2d(&tm_w, wb + bx * BoxGeom<WES>::kBoxBytes + quarter * 32 * BoxGeom<WES>::kPitch,
                             cc + bx * BoxGeom<WES>::kBoxCols, rr, pol);
            if constexpr (NMOM > 0) {
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SES>::kBoxes; ++bx)
                if (cc + bx * BoxGeom<SES>::kBoxCols < p.H)
                  tma_store_2d(&tm_m, mb + bx * BoxGeom<SES>::kBoxBytes + quarter * 32 * BoxGeom<SES>::kPitch,
                               cc + bx * BoxGeom<SES>::kBoxCols, rr, pol);
            }
            if constexpr (NMOM > 1) {
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SES>::kBoxes; ++bx)
                if (cc + bx * BoxGeom<SES>::kBoxCols < p.H)
                  tma_store_2d(&tm_v, vb + bx * BoxGeom<SES>::kBoxBytes + quarter * 32 * BoxGeom<SES>::kPitch,
                               cc + bx * BoxGeom<SES>::kBoxCols, rr, pol);
            }
          }
          tma_store_commit();
          tma_store_wait_read<0>();          // the stage may be refilled once the engine has read it
          mbar_arrive(&ctrl->st_empty[s]);
        }
        __syncwarp();
      }
      if (!ok) break;
      // all tcgen05.ld of this warp for this accumulator have completed
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctrl->acc_empty[buf]);
    }
    if (lane == 0) tma_store_wait_all<0>();
    if constexpr (ST == ST_FP8_TENSOR) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        amax_m_t = fmaxf(amax_m_t, __shfl_xor_sync(0xffffffffu, amax_m_t, o));
        amax_v_t = fmaxf(amax_v_t, __shfl_xor_sync(0xffffffffu, amax_v_t, o));
      }
      if (lane == 0) {
        // non-negative floats order like their bit patterns
        atomicMax(reinterpret_cast<unsigned int*>(p.m_absmax), __float_as_uint(amax_m_t));
        atomicMax(reinterpret_cast<unsigned int*>(p.v_absmax), __float_as_uint(amax_v_t));
      }
    }
  }

done:
  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // error path: give copies in flight a bounded time to land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace forge
