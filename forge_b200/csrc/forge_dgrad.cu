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
//
// Two extensions beyond the single product:
//   * up to MAX_SEG (dY_i, W_i) pairs are accumulated into one dX = sum_i dY_i W_i (the linears that
//     share an input -- q / k / v, gate / up -- have one input gradient): the producer walks the
//     segments' K ranges one after the other, the accumulator never leaves tensor memory;
//   * SCATTER: the row-sharded tensor-parallel mode's reduce-scatter of dX, fused into the GEMM.  The
//     columns of dX are cut into `world` feature blocks; the epilogue stores each 128 x 128 tile straight
//     into the receive buffer of the rank that owns its block -- slot [this rank] of that rank's
//     (world, BT, H / world) buffer -- with plain peer stores over NVLink (coalesced 256-byte runs from the
//     staging tile; no bulk-tensor copies and no multicast touch peer memory).  When the last CTA of the
//     launch has stored its last tile, one thread raises this rank's arrival word on every owner
//     (st.release.sys).  forge_reduce_slots on the owner waits (bounded) for all `world` arrival words and
//     adds the slots in rank order in fp32.  This replaces GEMM -> NCCL reduce-scatter
//     (src/fused_grad_optimizer/autograd.py:55 followed by a collective the reference does not have).
//   * FWD: the forward product of the same mode, Y = X W_r^T (src/fused_grad_optimizer/autograd.py:34) with
//     the all-gather of X fused into its consumer.  B = W_r is K-major here (H contiguous).  X arrives as
//     `world` feature blocks that the ranks push into this rank's gathered buffer (forge_push_block); each
//     block is one K segment, the own block first, and the producer waits (bounded) for a block's arrival
//     word only when it reaches that segment, so the MMAs on the blocks that are there overlap the
//     transfer of those that are not.  With the peer-store epilogue the output tiles go to every rank's
//     gathered Y (the all-gather of the row-sharded output), otherwise to local memory by TMA.
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>

#include "forge_host.h"
#include "forge_ptx.cuh"

namespace forge {

namespace dg {
constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 6;                       // single CTAs
constexpr int STAGES_PAIR = 7;                  // CTA pairs: each CTA stages its A rows and HALF of the B tile
constexpr int A_BYTES = BM * BK * 2;            // 16 KB, K-major, 128-byte swizzle
constexpr int B_BYTES = BK * BN * 2;            // 16 KB, two N-major slabs of 64 columns
constexpr int B_SLAB = 64 * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OUT_BYTES = BM * BN * 2;          // staging tile, two boxes of 64 columns
constexpr int CTRL_BYTES = 1024;
constexpr int STAGE_BYTES_PAIR = A_BYTES + B_BYTES / 2;
constexpr int SMEM_BYTES = CTRL_BYTES + 1024 + STAGES * STAGE_BYTES + OUT_BYTES;
constexpr int SMEM_BYTES_PAIR = CTRL_BYTES + 1024 + STAGES_PAIR * STAGE_BYTES_PAIR + OUT_BYTES;
constexpr int MAX_STAGES = STAGES_PAIR;
constexpr int THREADS = 256;
constexpr int ACC_BUFS = 4;
constexpr int TMEM_COLS = 512;
constexpr int MAX_SEG = 8;     // K segments: (dY_i, W_i) pairs accumulated into one dX (four at most through the C
                               // ABI), or the feature blocks of a gathered X
constexpr int MAX_RANKS = 8;
enum : int { ERR_OP_EMPTY = 201, ERR_OP_FULL = 202, ERR_ACC_EMPTY = 203, ERR_ACC_FULL = 204, ERR_ARRIVAL = 211 };

struct Ctrl {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[ACC_BUFS];
  uint64_t acc_empty[ACC_BUFS];
  uint32_t tmem_base;
  int abort_word;
};

struct alignas(64) Segment {
  CUtensorMap tm_a;     // dY_i: (BT, V_i), boxes of BK columns x BM rows
  CUtensorMap tm_b;     // W_i: (V_i, H), boxes of 64 columns x BK rows
  int num_kb;           // ceil(V_i / BK)
};

struct Params {
  int M, N;
  int tiles_m, tiles_n;
  int nseg, total_kb;
  int* status;
  // SCATTER
  int rank, world, block_cols;                 // block_cols = N / world, a multiple of BN
  int all_ranks;                               // 1: every tile goes to EVERY rank (slots are full width): a fused all-reduce
                                               // 2: every tile goes to every rank's ONE gathered matrix, at column
                                               //    push_col + n of rows push_pitch wide: an all-gather of the output
  int push_pitch, push_col;
  const uint32_t* seg_arrival[MAX_SEG];        // FWD: local arrival word of the block behind segment i, or NULL
  unsigned long long wait_ns;                  // FWD: how long the producer waits for a block
  int prefetch_kb;                             // the producer asks the L2 for B's tiles this many K blocks ahead
  uint8_t* slots[MAX_RANKS];                   // receive buffer of every rank, (world, M, block_cols) bf16
  uint32_t* arrivals[MAX_RANKS];               // arrival words of every rank, `world` each; [rank] is written here
  uint32_t* counter;                           // local: CTAs of this launch that have finished
  const uint32_t* epoch;                       // local device word: the value raised
  Segment seg[MAX_SEG];
};
}  // namespace dg

// CG = 2: a pair of CTAs (cluster of two, tcgen05 cta_group::2) shares a 256 x 128 tile.  Each CTA stages
// its own 128 rows of A and 64 of the tile's 128 columns of B (the MMA reads the two halves from the
// two CTAs' shared memory), so a stage is 24 KB instead of 32 KB for the same MMA work per SM.  The
// leader (rank 0) issues the MMAs; both CTAs' copies count on the leader's full barrier; its commits
// arrive on both CTAs' barriers (a barrier signal, not a data copy).
template <bool SCATTER, bool FWD, int CG>
__global__ void __launch_bounds__(dg::THREADS, 1)
forge_dgrad_kernel(const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ dg::Params p) {
  using namespace dg;
  constexpr int NSTAGE = CG == 2 ? STAGES_PAIR : STAGES;
  constexpr int STAGE_B = CG == 2 ? STAGE_BYTES_PAIR : STAGE_BYTES;
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int first_tile = (CG == 2) ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
  const int tile_step = static_cast<int>(gridDim.x) / CG;
  extern __shared__ uint8_t smem_raw[];
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem_raw);
  uint8_t* data = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + CTRL_BYTES + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* out_buf = data + NSTAGE * STAGE_B;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_word = &ctrl->abort_word;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&ctrl->full[i], 1); mbar_init(&ctrl->empty[i], 1); }
    for (int i = 0; i < ACC_BUFS; ++i) { mbar_init(&ctrl->acc_full[i], 1); mbar_init(&ctrl->acc_empty[i], 4 * CG); }
    ctrl->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_pair(&ctrl->tmem_base, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&ctrl->tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.seg[0].tm_a);
    prefetch_tmap(&p.seg[0].tm_b);
    if (!SCATTER) prefetch_tmap(&tm_out);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  // p.tiles_m counts tiles of BM * CG rows
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_a = policy_evict_last();    // dY is re-read by every column tile
      const uint64_t pol_b = policy_evict_first();   // W streams through once per row of tiles
      uint32_t it = 0;
      uint32_t arrived = 0;                          // FWD: segments whose block is known to be here
      for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
        // consecutive CTAs share a column panel of W: tile index runs over M fastest
        const int m0 = (tile % p.tiles_m) * (BM * CG) + static_cast<int>(cta_rank) * BM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int sg = 0; sg < p.nseg; ++sg) {
          const CUtensorMap* tm_a = &p.seg[sg].tm_a;
          const CUtensorMap* tm_b = &p.seg[sg].tm_b;
          const int nkb = p.seg[sg].num_kb;
          if constexpr (FWD) {
            const uint32_t* aw = p.seg_arrival[sg];
            if (aw != nullptr && !((arrived >> sg) & 1u)) {
              const uint32_t e = *p.epoch;
              const uint64_t t0 = global_timer_ns();
              for (uint32_t i = 0;; ++i) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(aw) : "memory");
                if (v == e) break;
                if ((i & 15u) == 15u && (*abort_word != 0 || global_timer_ns() - t0 > p.wait_ns)) {
                  atomicCAS(const_cast<int*>(abort_word), 0, ERR_ARRIVAL);
                  goto done;
                }
                __nanosleep(64);
              }
              fence_proxy_async_global();
              arrived |= 1u << sg;
            }
          }
          // W streams from HBM once and its latency is what the ring cannot cover: request its tiles a few
          // K blocks before the loads that need them (one request per 64 x 64-element box)
          auto prefetch_b = [&](int kb) {
            if constexpr (FWD) {
              if constexpr (CG == 2) {
                tma_prefetch_2d(tm_b, kb * BK, n0 + static_cast<int>(cta_rank) * 64);
              } else {
                tma_prefetch_2d(tm_b, kb * BK, n0);
              }
            } else {
              if constexpr (CG == 2) {
                tma_prefetch_2d(tm_b, n0 + static_cast<int>(cta_rank) * 64, kb * BK);
              } else {
                tma_prefetch_2d(tm_b, n0, kb * BK);
                tma_prefetch_2d(tm_b, n0 + 64, kb * BK);
              }
            }
          };
          const int pf = p.prefetch_kb;
          for (int kb = 0; kb < pf && kb < nkb; ++kb) prefetch_b(kb);
          for (int kb = 0; kb < nkb; ++kb, ++it) {
            const int s = it % NSTAGE;
            const uint32_t ph = (it / NSTAGE) & 1;
            if (pf > 0 && kb + pf < nkb) prefetch_b(kb + pf);
            if (!mbar_wait(&ctrl->empty[s], ph ^ 1, abort_word, ERR_OP_EMPTY)) goto done;
            uint8_t* a = data + s * STAGE_B;
            uint8_t* b = a + A_BYTES;
            // rows / columns past the end of a segment are zero-filled and add nothing
            if constexpr (CG == 2) {
              // both CTAs' copies count on the LEADER's barrier; the leader expects the bytes of both
              const uint32_t full_leader = map_to_cta(smem_u32(&ctrl->full[s]), 0);
              if (cta_rank == 0) mbar_expect_tx(&ctrl->full[s], 2 * STAGE_BYTES_PAIR);
              const int nh = n0 + static_cast<int>(cta_rank) * 64;        // this CTA's half of the tile's columns
              tma_load_2d_pair(a, tm_a, full_leader, kb * BK, m0, pol_a);
              if constexpr (FWD) tma_load_2d_pair(b, tm_b, full_leader, kb * BK, nh, pol_b);   // 64 rows of W_r, K-major
              else tma_load_2d_pair(b, tm_b, full_leader, nh, kb * BK, pol_b);
            } else {
              mbar_expect_tx(&ctrl->full[s], STAGE_BYTES);
              tma_load_2d(a, tm_a, &ctrl->full[s], kb * BK, m0, pol_a);
              if constexpr (FWD) {
                tma_load_2d(b, tm_b, &ctrl->full[s], kb * BK, n0, pol_b);          // 128 rows of W_r, K-major
              } else {
                tma_load_2d(b, tm_b, &ctrl->full[s], n0, kb * BK, pol_b);
                tma_load_2d(b + B_SLAB, tm_b, &ctrl->full[s], n0 + 64, kb * BK, pol_b);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * CG, BN, false, !FWD);
      uint32_t it = 0, tile_it = 0;
      for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++tile_it) {
        const int buf = tile_it % ACC_BUFS;
        const uint32_t aph = (tile_it / ACC_BUFS) & 1;
        if (!mbar_wait(&ctrl->acc_empty[buf], aph ^ 1, abort_word, ERR_ACC_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.total_kb; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          if (!mbar_wait(&ctrl->full[s], ph, abort_word, ERR_OP_FULL)) goto done;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(data + s * STAGE_B);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A (K-major): 16 K-elements further = 32 bytes inside the swizzle atom; 8-row groups
            // of M are 1024 bytes apart.  B (N-major): 16 K-rows further = two 1024-byte atoms;
            // 64-column slabs are B_SLAB bytes apart.
            const uint64_t da = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            // FWD: B is K-major like A (128 rows of W_r, 8-row groups 1024 bytes apart)
            const uint64_t db = FWD ? make_smem_desc_sw128(b_addr + k * 32, 16, 1024)
                                    : make_smem_desc_sw128(b_addr + k * 2048, B_SLAB, 1024);
            if constexpr (CG == 2) umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // frees the stage in both CTAs of a pair
          if constexpr (CG == 2) umma_commit_pair(&ctrl->empty[s], 3);
          else umma_commit(&ctrl->empty[s]);
        }
        if constexpr (CG == 2) umma_commit_pair(&ctrl->acc_full[buf], 3);
        else umma_commit(&ctrl->acc_full[buf]);
      }
    }
  } else if (warp >= 4) {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint64_t pol = policy_evict_last();   // dX is consumed by the next backward kernel
    uint32_t tile_it = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++tile_it) {
      const int m0 = (tile % p.tiles_m) * (BM * CG) + static_cast<int>(cta_rank) * BM;
      const int n0 = (tile / p.tiles_m) * BN;
      const int buf = tile_it % ACC_BUFS;
      const uint32_t aph = (tile_it / ACC_BUFS) & 1;
      bool ok = mbar_wait(&ctrl->acc_full[buf], aph, abort_word, ERR_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // the previous tile's store of this warp's rows must have been read out of the staging tile
      if constexpr (!SCATTER) {
        if (lane == 0) tma_store_wait_read<0>();
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + c * 32, acc);
        tmem_ld_wait();
        if (p.total_kb == 0) {
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
      if constexpr (!SCATTER) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->acc_empty[buf]), 0));
          else mbar_arrive(&ctrl->acc_empty[buf]);
          const int rr = m0 + quarter * 32;
          if (rr < p.M) {
            if (n0 < p.N) tma_store_2d(&tm_out, out_buf + quarter * 32 * 128, n0, rr, pol);
            if (n0 + 64 < p.N) tma_store_2d(&tm_out, out_buf + BM * 128 + quarter * 32 * 128, n0 + 64, rr, pol);
          }
          tma_store_commit();
        }
        __syncwarp();
      } else {
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->acc_empty[buf]), 0));
          else mbar_arrive(&ctrl->acc_empty[buf]);
        }
        // This warp's 32 rows of the staging tile go to the owner of the tile's feature block: slot
        // [this rank] of its receive buffer, row m, column n - owner * block_cols.  Two rows per
        // instruction, sixteen lanes x 16 bytes = one 256-byte run per row.
        // (all_ranks: the tile goes to every rank's slot [this rank], which is then N columns wide)
        const int piece = lane & 15, bx = piece >> 3, pc = piece & 7;
        // (all_ranks == 2: to every rank's single gathered matrix, at this rank's column offset)
        const int first = p.all_ranks ? 0 : n0 / p.block_cols;
        const int last = p.all_ranks ? p.world - 1 : first;
        const int pitch = p.all_ranks == 2 ? p.push_pitch : p.all_ranks ? p.N : p.block_cols;     // columns of a slot row
        const int col = p.all_ranks == 2 ? p.push_col + n0 : p.all_ranks ? n0 : n0 - first * p.block_cols;
        const size_t slot_row0 = p.all_ranks == 2 ? 0 : static_cast<size_t>(p.rank) * p.M;
        for (int owner = first; owner <= last; ++owner) {
          uint8_t* dst = p.slots[owner] + (slot_row0 * pitch + col) * 2;
#pragma unroll 4
          for (int rr = 0; rr < 32; rr += 2) {
            const int row = quarter * 32 + rr + (lane >> 4);
            const uint4 v = *reinterpret_cast<const uint4*>(out_buf + bx * (BM * 128) + row * 128 + ((pc ^ (row & 7)) << 4));
            if (m0 + row < p.M && n0 + piece * 8 < p.N)
              *reinterpret_cast<uint4*>(dst + static_cast<size_t>(m0 + row) * pitch * 2 + piece * 16) = v;
          }
        }
        __syncwarp();
      }
    }
    if constexpr (!SCATTER) {
      if (lane == 0) tma_store_wait_all<0>();
    } else {
      __threadfence_system();     // this thread's peer stores are visible system-wide before the CTA reports
    }
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
  if constexpr (SCATTER) {
    // (the barrier above orders every epilogue warp's stores and fences before this)
    if (threadIdx.x == 0 && *abort_word == 0) {
      const uint32_t done = atomicAdd(p.counter, 1u);
      if (done == gridDim.x - 1) {
        // last CTA of the launch: everyone's tiles are out; tell every owner that this rank's slot is complete
        __threadfence_system();
        *p.counter = 0u;                         // ready for the next launch that uses this word
        const uint32_t e = *p.epoch;
        for (int o = 0; o < p.world; ++o)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.arrivals[o] + p.rank), "r"(e) : "memory");
      }
    }
  }
  // a pair leaves together: the peer's shared memory and barriers stay valid until both are done
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[m, c] = sum over src = 0 .. world-1 of slot[src][m, c], added in that order in fp32, after every
// source rank's arrival word has reached the epoch.  One thread per CTA waits (bounded, like every wait
// of this library); a wait that runs out writes ERR_ARRIVAL to the status word and the CTA leaves its
// part of `out` untouched.
__global__ void __launch_bounds__(256)
forge_reduce_slots_kernel(const uint8_t* __restrict__ slots, const uint32_t* arrivals, const uint32_t* epoch,
                          __nv_bfloat16* __restrict__ out, int M, int S, long long ld_out, int world, int* status,
                          unsigned long long limit_ns, int n_slots, long long ld_slot) {
  // n_slots = world, ld_slot = S: the sum of the ranks' slots.  n_slots = 1: a copy of one gathered
  // matrix (row pitch ld_slot) once all `world` arrival words are there.
  __shared__ int ok;
  if (threadIdx.x == 0) {
    const uint32_t e = *epoch;
    int good = 1;
    const uint64_t t0 = global_timer_ns();
    for (int src = 0; src < world && good; ++src) {
      for (uint32_t i = 0;; ++i) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(arrivals + src) : "memory");
        if (v == e) break;
        if ((i & 15u) == 15u && global_timer_ns() - t0 > limit_ns) { good = 0; break; }
        __nanosleep(64);
      }
    }
    if (!good && status != nullptr) atomicCAS(status, 0, dg::ERR_ARRIVAL);
    ok = good;
  }
  __syncthreads();
  if (!ok) return;
  const long long pieces_per_row = S / 8;
  const long long total = static_cast<long long>(M) * pieces_per_row;
  const size_t slot_bytes = static_cast<size_t>(M) * ld_slot * 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / pieces_per_row, pc = i - m * pieces_per_row;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int src = 0; src < n_slots; ++src) {
      const uint4 q = *reinterpret_cast<const uint4*>(slots + src * slot_bytes + (m * ld_slot + pc * 8) * 2);
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += __uint_as_float(u[k] << 16);
        acc[2 * k + 1] += __uint_as_float(u[k] & 0xFFFF0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[k]) : "f"(acc[2 * k + 1]), "f"(acc[2 * k]));
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(out) + (m * ld_out + pc * 8) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace forge

using namespace forge;

namespace {

// validation, tensor maps of the segments and launch shared by the two entry points
template <bool SCATTER, bool FWD = false>
int launch_dgrad(const ForgeDgradSegment* segs, int nseg, void* dX, int64_t BT, int64_t H, int64_t ld_dx, dg::Params& p,
                 int32_t* status, cudaStream_t stream) {
  using namespace forge::dg;
  if (BT < 0 || H < 0 || nseg < 0) return fail(FORGE_ERR_INVALID_ARG, "negative dimension");
  if (nseg > (FWD ? MAX_SEG : 4)) return fail(FORGE_ERR_INVALID_ARG, "at most %d K segments per launch (got %d)", FWD ? MAX_SEG : 4, nseg);
  if (BT == 0 || H == 0) return FORGE_OK;
  if (nseg > 0 && segs == nullptr) return fail(FORGE_ERR_INVALID_ARG, "segments pointer is NULL");
  if (BT > (1 << 28) || H > (1ll << 30)) return fail(FORGE_ERR_SHAPE, "dimension too large");
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  if (di->cc_major != 10) return fail(FORGE_ERR_DEVICE, "device has compute capability %d.%d; sm_100 is required", di->cc_major, di->cc_minor);
  CUtensorMap tm_out;
  memset(&tm_out, 0, sizeof(tm_out));
  int rc;
  if (!SCATTER) {
    if (dX == nullptr) return fail(FORGE_ERR_INVALID_ARG, "dX is NULL");
    if ((rc = encode_tmap_2d(&tm_out, dX, 2, true, BT, H, ld_dx, 64, 32, 128)) != FORGE_OK) return rc;
  }
  // CTA pairs (FORGE_DGRAD_PAIRS=1) when there is more than one 128-row tile to pair up.  Off by default:
  // measured at BT = 512 they run at the rate of single CTAs, with seven or eight stages.
  static const bool pairs_allowed = [] {
    const char* e = getenv("FORGE_DGRAD_PAIRS");
    return e != nullptr && e[0] == '1';
  }();
  const int cg = (pairs_allowed && BT > BM) ? 2 : 1;
  static const int prefetch_kb = [] {
    const char* e = getenv("FORGE_DGRAD_PREFETCH");
    const int v = e != nullptr ? atoi(e) : 0;     // measured: no gain at 8 / 16 / 32 blocks ahead
    return v < 0 ? 0 : (v > 64 ? 64 : v);
  }();
  p.prefetch_kb = prefetch_kb;
  p.M = static_cast<int>(BT);
  p.N = static_cast<int>(H);
  p.tiles_m = static_cast<int>((BT + BM * cg - 1) / (BM * cg));
  p.tiles_n = static_cast<int>((H + BN - 1) / BN);
  p.nseg = 0;
  p.total_kb = 0;
  p.status = status;
  for (int i = 0; i < nseg; ++i) {
    const ForgeDgradSegment& g = segs[i];
    if (g.V < 0 || g.V > (1ll << 30)) return fail(FORGE_ERR_INVALID_ARG, "segment %d: bad V", i);
    if (g.V == 0) continue;
    if (g.dY == nullptr || g.W == nullptr) return fail(FORGE_ERR_INVALID_ARG, "segment %d: null pointer", i);
    p.seg_arrival[p.nseg] = p.seg_arrival[i];      // (FWD) follows its segment when empty ones are dropped
    Segment& sg = p.seg[p.nseg++];
    if ((rc = encode_tmap_2d(&sg.tm_a, g.dY, 2, true, BT, g.V, g.ld_dy, BK, BM, 128)) != FORGE_OK) return rc;
    if (FWD) {   // W_r block: H rows (the output columns) of g.V contiguous K elements; a pair's CTA takes 64 rows
      if ((rc = encode_tmap_2d(&sg.tm_b, g.W, 2, true, H, g.V, g.ld_w, BK, BN / cg, 128)) != FORGE_OK) return rc;
    } else {
      if ((rc = encode_tmap_2d(&sg.tm_b, g.W, 2, true, g.V, H, g.ld_w, 64, BK, 128)) != FORGE_OK) return rc;
    }
    sg.num_kb = static_cast<int>((g.V + BK - 1) / BK);
    p.total_kb += sg.num_kb;
  }
  if (p.nseg == 0) {   // nothing to multiply: the maps are never used, pass valid memory anyway
    p.seg[0].tm_a = tm_out;
    p.seg[0].tm_b = tm_out;
    p.seg[0].num_kb = 0;
  }
  static std::atomic<bool> attr_set[64][2];   // per device and form: the shared-memory opt-in has been made
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem = cg == 2 ? SMEM_BYTES_PAIR : SMEM_BYTES;
  if (dev >= 0 && dev < 64 && !attr_set[dev][cg - 1].load(std::memory_order_acquire)) {
    cudaError_t e = cg == 2 ? cudaFuncSetAttribute(forge_dgrad_kernel<SCATTER, FWD, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                            : cudaFuncSetAttribute(forge_dgrad_kernel<SCATTER, FWD, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set[dev][cg - 1].store(true, std::memory_order_release);
  }
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  cudaError_t e;
  if (cg == 2) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * static_cast<unsigned>(std::min<int64_t>(tiles, di->sm_count / 2)), 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, forge_dgrad_kernel<SCATTER, FWD, 2>, tm_out, p);
  } else {
    const int grid = static_cast<int>(std::min<int64_t>(tiles, di->sm_count));
    forge_dgrad_kernel<SCATTER, FWD, 1><<<grid, THREADS, smem, stream>>>(tm_out, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "dgrad kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

}  // namespace

extern "C" int forge_dgrad(const void* dY, const void* W, void* dX, int64_t BT, int64_t V, int64_t H,
                           int64_t ld_dy, int64_t ld_w, int64_t ld_dx, int32_t* status, void* cuda_stream) {
  if (V < 0) return fail(FORGE_ERR_INVALID_ARG, "negative dimension");
  ForgeDgradSegment seg = {dY, W, V, ld_dy, ld_w};
  return forge_dgrad_sum(&seg, 1, dX, BT, H, ld_dx, status, cuda_stream);
}

extern "C" int forge_dgrad_sum(const ForgeDgradSegment* segments, int32_t count, void* dX, int64_t BT, int64_t H,
                               int64_t ld_dx, int32_t* status, void* cuda_stream) {
  dg::Params p;
  memset(&p, 0, sizeof(p));
  return launch_dgrad<false>(segments, count, dX, BT, H, ld_dx, p, status, static_cast<cudaStream_t>(cuda_stream));
}

extern "C" int forge_dgrad_scatter(const ForgeDgradScatterArgs* args, void* cuda_stream) {
  using namespace forge::dg;
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_dgrad_scatter: args is NULL");
  const ForgeDgradScatterArgs& a = *args;
  if (a.world < 1 || a.world > MAX_RANKS || a.rank < 0 || a.rank >= a.world)
    return fail(FORGE_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", a.rank, a.world, MAX_RANKS);
  if (a.H <= 0 || a.H % 8 != 0 || (!a.all_ranks && (a.H % a.world != 0 || (a.H / a.world) % BN != 0)))
    return fail(FORGE_ERR_SHAPE, "H (%lld) must split into %d feature blocks that are multiples of %d columns "
                "(any multiple of 8 when every rank receives everything)", (long long)a.H, a.world, BN);
  if (a.slots == nullptr || a.arrivals == nullptr || a.counter == nullptr || a.epoch == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_dgrad_scatter: slots / arrivals / counter / epoch is NULL");
  dg::Params p;
  memset(&p, 0, sizeof(p));
  p.rank = a.rank;
  p.world = a.world;
  p.block_cols = static_cast<int>(a.all_ranks ? a.H : a.H / a.world);
  p.all_ranks = a.all_ranks ? 1 : 0;
  for (int r = 0; r < a.world; ++r) {
    if (a.slots[r] == nullptr || a.arrivals[r] == nullptr || !aligned16(a.slots[r]))
      return fail(FORGE_ERR_INVALID_ARG, "receive buffer or arrival words of rank %d are NULL or misaligned", r);
    p.slots[r] = static_cast<uint8_t*>(a.slots[r]);
    p.arrivals[r] = a.arrivals[r];
  }
  p.counter = a.counter;
  p.epoch = a.epoch;
  return launch_dgrad<true>(a.segments, a.count, nullptr, a.BT, a.H, 0, p, a.status, static_cast<cudaStream_t>(cuda_stream));
}

// time a reduce waits for its arrivals before it gives up (nanoseconds of the global timer)
static std::atomic<uint64_t> g_arrival_wait_ns{FORGE_WAIT_NS};

extern "C" int forge_set_arrival_wait_ns(uint64_t ns) {
  if (ns == 0 || ns > 60000000000ull) return fail(FORGE_ERR_INVALID_ARG, "arrival wait must be 1 ns .. 60 s");
  g_arrival_wait_ns.store(ns);
  return FORGE_OK;
}

extern "C" int forge_reduce_slots(const void* slots, const uint32_t* arrivals, const uint32_t* epoch, void* out, int64_t BT,
                                  int64_t block_cols, int64_t ld_out, int32_t world, int32_t* status, void* cuda_stream) {
  if (slots == nullptr || arrivals == nullptr || epoch == nullptr || out == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_reduce_slots: null pointer");
  if (world < 1 || world > dg::MAX_RANKS || BT < 0 || block_cols <= 0 || block_cols % 8 != 0 || ld_out % 8 != 0 ||
      !aligned16(slots) || !aligned16(out))
    return fail(FORGE_ERR_INVALID_ARG, "forge_reduce_slots: bad shape, world size or alignment");
  if (BT == 0) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  const int64_t pieces = BT * (block_cols / 8);
  const int grid = static_cast<int>(std::min<int64_t>((pieces + 255) / 256, 2 * di->sm_count));
  forge_reduce_slots_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(slots), arrivals, epoch, static_cast<__nv_bfloat16*>(out), static_cast<int>(BT),
      static_cast<int>(block_cols), ld_out, world, status, g_arrival_wait_ns.load(), world, block_cols);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "reduce kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

extern "C" int forge_collect(const void* gathered, int64_t ld_gathered, const uint32_t* arrivals, const uint32_t* epoch,
                             void* out, int64_t BT, int64_t cols, int64_t ld_out, int32_t world, int32_t* status,
                             void* cuda_stream) {
  if (gathered == nullptr || arrivals == nullptr || epoch == nullptr || out == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_collect: null pointer");
  if (world < 1 || world > dg::MAX_RANKS || BT < 0 || cols <= 0 || cols % 8 != 0 || ld_out % 8 != 0 || ld_gathered % 8 != 0 ||
      ld_gathered < cols || !aligned16(gathered) || !aligned16(out))
    return fail(FORGE_ERR_INVALID_ARG, "forge_collect: bad shape, world size or alignment");
  if (BT == 0) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  const int64_t pieces = BT * (cols / 8);
  const int grid = static_cast<int>(std::min<int64_t>((pieces + 255) / 256, 2 * di->sm_count));
  forge_reduce_slots_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
      static_cast<const uint8_t*>(gathered), arrivals, epoch, static_cast<__nv_bfloat16*>(out), static_cast<int>(BT),
      static_cast<int>(cols), ld_out, world, status, g_arrival_wait_ns.load(), 1, ld_gathered);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "collect kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

namespace forge {
// this rank's (M, cols) block -> column `col` of every rank's (M, ld_dst) matrix; the last CTA raises
// arrival word [rank] on every rank (same protocol as the GEMM's peer-store epilogue)
struct PushParams {
  const uint8_t* src;
  long long ld_src, ld_dst, col;
  int M, cols, rank, world;
  uint8_t* dst[dg::MAX_RANKS];
  uint32_t* arrivals[dg::MAX_RANKS];
  uint32_t* counter;
  const uint32_t* epoch;
};

__global__ void __launch_bounds__(256)
forge_push_block_kernel(const __grid_constant__ PushParams p) {
  const long long pieces_per_row = p.cols / 8;
  const long long total = static_cast<long long>(p.M) * pieces_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / pieces_per_row, pc = i - m * pieces_per_row;
    const uint4 v = *reinterpret_cast<const uint4*>(p.src + (m * p.ld_src + pc * 8) * 2);
    for (int o = 0; o < p.world; ++o)
      *reinterpret_cast<uint4*>(p.dst[o] + (m * p.ld_dst + p.col + pc * 8) * 2) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(p.counter, 1u);
    if (done == gridDim.x - 1) {
      __threadfence_system();
      *p.counter = 0u;
      const uint32_t e = *p.epoch;
      for (int o = 0; o < p.world; ++o)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.arrivals[o] + p.rank), "r"(e) : "memory");
    }
  }
}
}  // namespace forge

extern "C" int forge_push_block(const void* src, int64_t BT, int64_t cols, int64_t ld_src, void* const* dst, int64_t col,
                                int64_t ld_dst, uint32_t* const* arrivals, uint32_t* counter, const uint32_t* epoch,
                                int32_t rank, int32_t world, int32_t* status, void* cuda_stream) {
  (void)status;
  if (src == nullptr || dst == nullptr || arrivals == nullptr || counter == nullptr || epoch == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_push_block: null pointer");
  if (world < 1 || world > dg::MAX_RANKS || rank < 0 || rank >= world)
    return fail(FORGE_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", rank, world, dg::MAX_RANKS);
  if (BT < 0 || cols <= 0 || cols % 8 != 0 || col < 0 || col % 8 != 0 || ld_src % 8 != 0 || ld_dst % 8 != 0 ||
      col + cols > ld_dst || ld_src < cols || !aligned16(src))
    return fail(FORGE_ERR_INVALID_ARG, "forge_push_block: bad shape or alignment");
  forge::PushParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < world; ++r) {
    if (dst[r] == nullptr || arrivals[r] == nullptr || !aligned16(dst[r]))
      return fail(FORGE_ERR_INVALID_ARG, "gathered matrix or arrival words of rank %d are NULL or misaligned", r);
    p.dst[r] = static_cast<uint8_t*>(dst[r]);
    p.arrivals[r] = arrivals[r];
  }
  if (BT == 0) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  p.src = static_cast<const uint8_t*>(src);
  p.ld_src = ld_src;
  p.ld_dst = ld_dst;
  p.col = col;
  p.M = static_cast<int>(BT);
  p.cols = static_cast<int>(cols);
  p.rank = rank;
  p.world = world;
  p.counter = counter;
  p.epoch = epoch;
  const int64_t pieces = BT * (cols / 8);
  const int grid = static_cast<int>(std::min<int64_t>((pieces + 255) / 256, di->sm_count));
  forge::forge_push_block_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "push kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

extern "C" int forge_linear_gathered(const ForgeLinearGatheredArgs* args, void* cuda_stream) {
  using namespace forge::dg;
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_linear_gathered: args is NULL");
  const ForgeLinearGatheredArgs& a = *args;
  if (a.world < 1 || a.world > MAX_RANKS || a.rank < 0 || a.rank >= a.world)
    return fail(FORGE_ERR_INVALID_ARG, "rank %d of %d (at most %d ranks)", a.rank, a.world, MAX_RANKS);
  if (a.X == nullptr || a.W == nullptr || a.epoch == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_linear_gathered: X / W / epoch is NULL");
  if (a.H <= 0 || a.H % (8 * a.world) != 0)
    return fail(FORGE_ERR_SHAPE, "H (%lld) must split into %d feature blocks that are multiples of 8 columns", (long long)a.H, a.world);
  if (a.V_r < 0 || a.V_r % 8 != 0) return fail(FORGE_ERR_SHAPE, "V_r (%lld) must be a multiple of 8", (long long)a.V_r);
  const int64_t blk = a.H / a.world;
  Params p;
  memset(&p, 0, sizeof(p));
  p.rank = a.rank;
  p.world = a.world;
  p.epoch = a.epoch;
  p.wait_ns = g_arrival_wait_ns.load();
  // K segments = feature blocks, the own block first, then the ranks after this one in ring order
  ForgeDgradSegment segs[MAX_SEG];
  for (int i = 0; i < a.world; ++i) {
    const int src = (a.rank + i) % a.world;
    segs[i].dY = static_cast<const uint8_t*>(a.X) + src * blk * 2;
    segs[i].W = static_cast<const uint8_t*>(a.W) + src * blk * 2;
    segs[i].V = blk;
    segs[i].ld_dy = a.ld_x;
    segs[i].ld_w = a.ld_w;
    p.seg_arrival[i] = (a.x_arrivals != nullptr && src != a.rank) ? a.x_arrivals + src : nullptr;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (a.y != nullptr)
    return launch_dgrad<false, true>(segs, a.world, a.y, a.BT, a.V_r, a.ld_y, p, a.status, stream);
  if (a.y_dst == nullptr || a.y_arrivals == nullptr || a.y_counter == nullptr)
    return fail(FORGE_ERR_INVALID_ARG, "forge_linear_gathered: neither a local output nor the pushed form's buffers");
  if (a.y_col < 0 || a.y_col % 8 != 0 || a.y_pitch % 8 != 0 || a.y_col + a.V_r > a.y_pitch)
    return fail(FORGE_ERR_SHAPE, "pushed output: column offset / pitch must be multiples of 8 and hold V_r columns");
  for (int r = 0; r < a.world; ++r) {
    if (a.y_dst[r] == nullptr || a.y_arrivals[r] == nullptr || !aligned16(a.y_dst[r]))
      return fail(FORGE_ERR_INVALID_ARG, "gathered output or arrival words of rank %d are NULL or misaligned", r);
    p.slots[r] = static_cast<uint8_t*>(a.y_dst[r]);
    p.arrivals[r] = a.y_arrivals[r];
  }
  p.counter = a.y_counter;
  p.all_ranks = 2;
  p.push_pitch = static_cast<int>(a.y_pitch);
  p.push_col = static_cast<int>(a.y_col);
  p.block_cols = static_cast<int>(a.V_r);
  return launch_dgrad<true, true>(segs, a.world, nullptr, a.BT, a.V_r, 0, p, a.status, stream);
}
