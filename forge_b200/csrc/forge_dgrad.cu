// dX = dY W : (BT, V) x (V, H) -> (BT, H), bf16 operands, fp32 accumulation in tensor memory, bf16
// output.  Replaces `grad_input = grad_output @ weight` (src/fused_grad_optimizer/autograd.py:55).
// It must be enqueued before the fused update of the same W on the same stream.
//
// GEMM view: M = BT, N = H, K = V.  A = dY is K-major (V contiguous), B = W is N-major (H
// contiguous), so neither operand is transposed in memory.  One persistent CTA per SM:
//   warp 0      TMA producer (128 x 64 panel of dY, 64 x 128 panel of W per stage)
//   warp 1      tensor-memory owner + tcgen05.mma issuer
//   warps 4-7   epilogue: tcgen05.ld, fp32 -> bf16, swizzled staging tile, one TMA store per warp
// Four 128 x 128 fp32 accumulators live in tensor memory, so the MMAs of the next tile start while
// the previous tile is still being written out.
#include <algorithm>
#include <atomic>

#include "forge_host.h"
#include "forge_ptx.cuh"

namespace forge {

namespace dg {
constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB, K-major, 128-byte swizzle
constexpr int B_BYTES = BK * BN * 2;            // 16 KB, two N-major slabs of 64 columns
constexpr int B_SLAB = 64 * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OUT_BYTES = BM * BN * 2;          // staging tile, two boxes of 64 columns
constexpr int CTRL_BYTES = 1024;
constexpr int SMEM_BYTES = CTRL_BYTES + 1024 + STAGES * STAGE_BYTES + OUT_BYTES;
constexpr int THREADS = 256;
constexpr int ACC_BUFS = 4;
constexpr int TMEM_COLS = 512;
enum : int { ERR_OP_EMPTY = 201, ERR_OP_FULL = 202, ERR_ACC_EMPTY = 203, ERR_ACC_FULL = 204 };

struct Ctrl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[ACC_BUFS];
  uint64_t acc_empty[ACC_BUFS];
  uint32_t tmem_base;
  int abort_word;
};

struct Params {
  int M, N, K;
  int tiles_m, tiles_n, num_kb;
  int* status;
};
}  // namespace dg

__global__ void __launch_bounds__(dg::THREADS, 1)
forge_dgrad_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_out, const dg::Params p) {
  using namespace dg;
  extern __shared__ uint8_t smem_raw[];
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw);
  uint8_t* data = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + CTRL_BYTES + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* out_buf = data + STAGES * STAGE_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_word = &ctrl->abort_word;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&ctrl->full[i], 1); mbar_init(&ctrl->empty[i], 1); }
    for (int i = 0; i < ACC_BUFS; ++i) { mbar_init(&ctrl->acc_full[i], 1); mbar_init(&ctrl->acc_empty[i], 4); }
    ctrl->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) { prefetch_tmap(&tm_a); prefetch_tmap(&tm_b); prefetch_tmap(&tm_out); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_a = policy_evict_last();    // dY is re-read by every column tile
      const uint64_t pol_b = policy_evict_first();   // W streams through once per row of tiles
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        // consecutive CTAs share a column panel of W: tile index runs over M fastest
        const int m0 = (tile % p.tiles_m) * BM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctrl->empty[s], ph ^ 1, abort_word, ERR_OP_EMPTY)) goto done;
          uint8_t* a = data + s * STAGE_BYTES;
          uint8_t* b = a + A_BYTES;
          mbar_expect_tx(&ctrl->full[s], STAGE_BYTES);
          tma_load_2d(a, &tm_a, &ctrl->full[s], kb * BK, m0, pol_a);
          tma_load_2d(b, &tm_b, &ctrl->full[s], n0, kb * BK, pol_b);
          tma_load_2d(b + B_SLAB, &tm_b, &ctrl->full[s], n0 + 64, kb * BK, pol_b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, true);
      uint32_t it = 0, tile_it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_it) {
        const int buf = tile_it % ACC_BUFS;
        const uint32_t aph = (tile_it / ACC_BUFS) & 1;
        if (!mbar_wait(&ctrl->acc_empty[buf], aph ^ 1, abort_word, ERR_ACC_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctrl->full[s], ph, abort_word, ERR_OP_FULL)) goto done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(data + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A (K-major): 16 K-elements further = 32 bytes inside the swizzle atom; 8-row groups
            // of M are 1024 bytes apart.  B (N-major): 16 K-rows further = two 1024-byte atoms;
            // 64-column slabs are B_SLAB bytes apart.
            const uint64_t da = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(b_addr + k * 2048, B_SLAB, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&ctrl->empty[s]);
        }
        umma_commit(&ctrl->acc_full[buf]);
      }
    }
  } else if (warp >= 4) {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint64_t pol = policy_evict_last();   // dX is consumed by the next backward kernel
    uint32_t tile_it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_it) {
      const int m0 = (tile % p.tiles_m) * BM;
      const int n0 = (tile / p.tiles_m) * BN;
      const int buf = tile_it % ACC_BUFS;
      const uint32_t aph = (tile_it / ACC_BUFS) & 1;
      bool ok = mbar_wait(&ctrl->acc_full[buf], aph, abort_word, ERR_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // the previous tile's store of this warp's rows must have been read out of the staging tile
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + c * 32, acc);
        tmem_ld_wait();
        if (p.num_kb == 0) {
#pragma unroll
          for (int k = 0; k < 32; ++k) acc[k] = 0u;
        }
        // columns [32c, 32c+32) -> box (c >> 1), 16-byte pieces 4*(c&1) .. +3 of the 128-byte row
        uint8_t* box = out_buf + (c >> 1) * (BM * 128) + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t u[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(acc[8 * j + 2 * i]), hi = __uint_as_float(acc[8 * j + 2 * i + 1]);
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u[i]) : "f"(hi), "f"(lo));
          }
          const int piece = 4 * (c & 1) + j;
          *reinterpret_cast<uint4*>(box + ((piece ^ (r & 7)) << 4)) = make_uint4(u[0], u[1], u[2], u[3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&ctrl->acc_empty[buf]);
        const int rr = m0 + quarter * 32;
        if (rr < p.M) {
          if (n0 < p.N) tma_store_2d(&tm_out, out_buf + quarter * 32 * 128, n0, rr, pol);
          if (n0 + 64 < p.N) tma_store_2d(&tm_out, out_buf + BM * 128 + quarter * 32 * 128, n0 + 64, rr, pol);
        }
        tma_store_commit();
      }
      __syncwarp();
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

done:
  // the single-lane roles leave their loops alone; bring every warp back together before the
  // CTA-wide barrier (an aligned barrier executed by a diverged warp is undefined)
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
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

using namespace forge;

extern "C" int forge_dgrad(const void* dY, const void* W, void* dX, int64_t BT, int64_t V, int64_t H,
                           int64_t ld_dy, int64_t ld_w, int64_t ld_dx, int32_t* status, void* cuda_stream) {
  using namespace forge::dg;
  if (BT < 0 || V < 0 || H < 0) return fail(FORGE_ERR_INVALID_ARG, "negative dimension");
  if (BT == 0 || H == 0) return FORGE_OK;
  if (dX == nullptr || (V > 0 && (dY == nullptr || W == nullptr))) return fail(FORGE_ERR_INVALID_ARG, "null pointer");
  if (BT > (1 << 28) || V > (1ll << 30) || H > (1ll << 30)) return fail(FORGE_ERR_SHAPE, "dimension too large");
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  if (di->cc_major != 10) return fail(FORGE_ERR_DEVICE, "device has compute capability %d.%d; sm_100 is required", di->cc_major, di->cc_minor);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  CUtensorMap tm_a, tm_b, tm_out;
  int rc;
  if ((rc = encode_tmap_2d(&tm_out, dX, 2, true, BT, H, ld_dx, 64, 32, 128)) != FORGE_OK) return rc;
  if (V > 0) {
    if ((rc = encode_tmap_2d(&tm_a, dY, 2, true, BT, V, ld_dy, BK, BM, 128)) != FORGE_OK) return rc;
    if ((rc = encode_tmap_2d(&tm_b, W, 2, true, V, H, ld_w, 64, BK, 128)) != FORGE_OK) return rc;
  } else {
    tm_a = tm_out;
    tm_b = tm_out;
  }
  Params p;
  p.M = static_cast<int>(BT);
  p.N = static_cast<int>(H);
  p.K = static_cast<int>(V);
  p.tiles_m = static_cast<int>((BT + BM - 1) / BM);
  p.tiles_n = static_cast<int>((H + BN - 1) / BN);
  p.num_kb = static_cast<int>((V + BK - 1) / BK);
  p.status = status;
  static std::atomic<bool> attr_set[64];   // per device: the shared-memory opt-in has been made
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(forge_dgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  const int grid = static_cast<int>(std::min<int64_t>(tiles, di->sm_count));
  forge_dgrad_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tm_a, tm_b, tm_out, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "dgrad kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}
