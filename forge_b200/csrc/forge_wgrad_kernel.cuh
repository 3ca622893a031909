// Fused weight-gradient + optimizer kernel for sm_100a.
//
//   dW[v,h] = sum_bt dY[bt,v] * X[bt,h]          (bf16 x bf16, fp32 accumulate in tensor memory)
//   (W, moments)[v,h] <- optimizer(W, moments, dW)   applied to the accumulator tile on chip
//
// No gradient tensor is written to global memory.  This replaces the reference's fused kernels
// (src/fused_grad_optimizer/kernel.py:212-317 AdamW, :122-205 SGD, :324-478 int8 moments,
// kernel_fp8_state.py:204-295 fp8 moments).  The reference launches one kernel per linear; one launch
// here updates a GROUP of up to MAX_GROUP weights of the same kernel configuration (say the q / k / v
// projections, or all seven projections of one or two decoder layers): the work units of the problems are
// numbered one after the other, the roles look up the problem a unit belongs to, and the pipelines
// (operand ring, state ring, accumulators) run on across problem boundaries, so the start-up and the
// ragged end of a launch are paid once per group instead of once per weight.
//
// Structure: one persistent CTA per SM, 12 warps.
//   warp 0      TMA producer of the dY / X panels (both operands are M/N-major in memory: dY is
//               (BT,V) with V contiguous, X is (BT,H) with H contiguous; no transpose is made)
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), frees it
//   warp 2      TMA producer of the W / moment sub-tiles (prefetched while the MMAs of the tile run)
//   warp 3      TMA store issuer: writes each updated sub-tile back and returns its stage to warp 2
//   warps 4-11  epilogue: two groups of four warps; group g handles the column chunks g, g+2, ...
//               of the 128 x 256 tile (chunks are 64 columns wide, 32 when a 64-column stage would
//               not fit four times).  Each thread owns one accumulator row: tcgen05.ld, fp32 update
//               against the staged W/moment rows in shared memory (in place), then the warp hands
//               the chunk to warp 3.  Issuing the bulk stores from the epilogue warps themselves
//               stalled them for 0.3-0.9 us per chunk behind the loads queued in the TMA unit.
// The ring of state stages has an even number of slots, so the chunks of group g always land in
// slots of parity g: every full/empty barrier then has a single consumer group that observes each
// of its phases, which is what makes waiting on the phase parity sound.
// Tensor memory holds two 128 x 256 fp32 accumulators, so the MMAs of tile i+1 overlap the
// epilogue of tile i.
//
// Work distribution: the grid has one cluster (a CTA, or a CTA pair) per work unit, units numbered
// row-major over the tiles.  Only as many clusters as fit on the GPU start; each of them, when it
// has queued the loads of its unit, asks the hardware (cluster launch control) for a unit whose
// cluster has not started yet, cancels that launch and does the unit itself.  SMs that run a
// little slower than the others (10 % was seen) simply take fewer units, and the units in flight
// at any moment stay neighbours in memory, so whole rows of W and of the moments stream from the
// same DRAM pages.  The scheduler is the operand producer of the (leading) CTA; it passes unit
// numbers to the other roles, and to the second CTA of a pair, through a four-slot queue in
// shared memory (st.async + mbarrier).  The last `p.num_units - p.split_from` units are
// 128-column halves of a tile: a weight with few tiles is cut that way to occupy more SMs.
#pragma once

#include "forge_ptx.cuh"
#include "forge_update.cuh"

namespace forge {

constexpr int TILE_M = 128;        // rows of W per tile (V direction)
constexpr int TILE_N = 256;        // columns of W per tile (H direction)
constexpr int UMMA_K = 16;
#ifndef FORGE_OP_BK
#define FORGE_OP_BK 32
#endif
#ifndef FORGE_OP_STAGES
#define FORGE_OP_STAGES 3
#endif
#ifndef FORGE_FILL_GATE_CHUNKS
#define FORGE_FILL_GATE_CHUNKS 2
#endif
#ifndef FORGE_MAX_STATE_STAGES
#define FORGE_MAX_STATE_STAGES 6
#endif
constexpr int OP_BK = FORGE_OP_BK;           // token rows per operand pipeline stage
constexpr int OP_STAGES = FORGE_OP_STAGES;   // operand pipeline depth
constexpr int EPI_WARP0 = 4;
// 1: sixteen epilogue warps for the block-quantised modes (see WgradCfg::kWide).  Off: measured slower
// (14336 x 4096 int8: 183 us against 160 us), although correct.
#ifndef FORGE_WIDE_EPILOGUE
#define FORGE_WIDE_EPILOGUE 0
#endif
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BUDGET = 227 * 1024;

// error codes written to the status word
enum : int {
  ERR_WAIT_OP_EMPTY = 101,
  ERR_WAIT_OP_FULL = 102,
  ERR_WAIT_ST_EMPTY = 103,
  ERR_WAIT_ST_FULL = 104,
  ERR_WAIT_ACC_EMPTY = 105,
  ERR_WAIT_ACC_FULL = 106,
  ERR_WAIT_ST_DONE = 107,
  ERR_WAIT_TQ_FULL = 108,
  ERR_WAIT_TQ_EMPTY = 109,
  ERR_WAIT_CLC = 110,
  ERR_WAIT_FILL_GATE = 111
};

// Geometry of one 128-row chunk of a tensor whose rows are RB bytes wide inside the chunk.
template <int RB>
struct BoxGeom;
template <>
struct BoxGeom<256> {  // two boxes of 128 bytes per row each, 128-byte swizzle (fp32, 64 columns)
  static constexpr int kBoxes = 2, kBoxRowBytes = 128, kPitch = 128, kBoxBytes = 128 * 128, kSwizzle = 128;
};
template <>
struct BoxGeom<128> {  // one box, 128 bytes per row, 128-byte swizzle
  static constexpr int kBoxes = 1, kBoxRowBytes = 128, kPitch = 128, kBoxBytes = 128 * 128, kSwizzle = 128;
};
template <>
struct BoxGeom<64> {  // one box, 64 bytes per row, 64-byte swizzle
  static constexpr int kBoxes = 1, kBoxRowBytes = 64, kPitch = 64, kBoxBytes = 128 * 64, kSwizzle = 64;
};
template <>
struct BoxGeom<0> {  // absent tensor
  static constexpr int kBoxes = 0, kBoxRowBytes = 16, kPitch = 0, kBoxBytes = 0, kSwizzle = 0;
};

__host__ __device__ constexpr int num_moments(int opt) {
  return opt == OPT_ADAMW ? 2 : (opt == OPT_SGD ? 0 : 1);
}
__host__ __device__ constexpr int state_elem_size(int st) {
  return st == ST_F32 ? 4 : (st == ST_BF16 ? 2 : (st == ST_NONE ? 0 : 1));
}

// byte offset of the 16-byte piece `j` of row `r` inside a chunk buffer with RB-byte rows
template <int RB>
__device__ __forceinline__ uint32_t piece_off(int r, int j) {
  if constexpr (RB == 256) {
    return (j >> 3) * BoxGeom<256>::kBoxBytes + r * 128 + (((j & 7) ^ (r & 7)) << 4);
  } else if constexpr (RB == 128) {
    return r * 128 + ((j ^ (r & 7)) << 4);
  } else {
    static_assert(RB == 64, "row bytes");
    return r * 64 + ((j ^ ((r >> 1) & 3)) << 4);
  }
}

// ---- 16-element row groups: raw 16-byte pieces <-> fp32 registers --------------------------------
// The raw pieces of the NEXT group are fetched before the current group is computed and stored
// (shared-memory loads cannot be hoisted over stores by the compiler, the swizzled addresses defeat
// its alias analysis), so load latency overlaps arithmetic.
template <int ES>
struct Raw16 {
  uint4 q[ES];   // 16 elements: one piece of codes, two of bf16, four of fp32
};

template <int ES, int RB>
__device__ __forceinline__ Raw16<ES> load_raw(const uint8_t* buf, int r, int g) {
  Raw16<ES> x;
#pragma unroll
  for (int p = 0; p < ES; ++p) x.q[p] = *reinterpret_cast<const uint4*>(buf + piece_off<RB>(r, ES * g + p));
  return x;
}

template <int ES, int RB>
__device__ __forceinline__ void store_raw(uint8_t* buf, int r, int g, const Raw16<ES>& x) {
#pragma unroll
  for (int p = 0; p < ES; ++p) *reinterpret_cast<uint4*>(buf + piece_off<RB>(r, ES * g + p)) = x.q[p];
}

template <int ES>
__device__ __forceinline__ void unpack16(const Raw16<ES>& x, float (&out)[16]) {
  if constexpr (ES == 4) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      out[4 * p + 0] = __uint_as_float(x.q[p].x); out[4 * p + 1] = __uint_as_float(x.q[p].y);
      out[4 * p + 2] = __uint_as_float(x.q[p].z); out[4 * p + 3] = __uint_as_float(x.q[p].w);
    }
  } else {
    static_assert(ES == 2, "float/bf16 only");
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const uint32_t u[4] = {x.q[p].x, x.q[p].y, x.q[p].z, x.q[p].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[8 * p + 2 * i + 0] = __uint_as_float(u[i] << 16);
        out[8 * p + 2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
      }
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

template <int ES>
__device__ __forceinline__ Raw16<ES> pack16(const float (&in)[16]) {
  Raw16<ES> x;
  if constexpr (ES == 4) {
#pragma unroll
    for (int p = 0; p < 4; ++p)
      x.q[p] = make_uint4(__float_as_uint(in[4 * p + 0]), __float_as_uint(in[4 * p + 1]),
                          __float_as_uint(in[4 * p + 2]), __float_as_uint(in[4 * p + 3]));
  } else {
    static_assert(ES == 2, "float/bf16 only");
#pragma unroll
    for (int p = 0; p < 2; ++p)
      x.q[p] = make_uint4(pack_bf16x2(in[8 * p + 0], in[8 * p + 1]), pack_bf16x2(in[8 * p + 2], in[8 * p + 3]),
                          pack_bf16x2(in[8 * p + 4], in[8 * p + 5]), pack_bf16x2(in[8 * p + 6], in[8 * p + 7]));
  }
  return x;
}

// one-byte codes: 64-column chunks only (row = 64 bytes)
__device__ __forceinline__ void ld16_bytes(const uint8_t* buf, int r, int g, uint32_t (&w)[4]) {
  const uint4 q = *reinterpret_cast<const uint4*>(buf + piece_off<64>(r, g));
  w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w;
}
__device__ __forceinline__ void st16_bytes(uint8_t* buf, int r, int g, const uint32_t (&w)[4]) {
  *reinterpret_cast<uint4*>(buf + piece_off<64>(r, g)) = make_uint4(w[0], w[1], w[2], w[3]);
}

// kernel parameters ------------------------------------------------------------------------------
constexpr int MAX_GROUP = 16;   // weights per launch (two decoder layers of seven projections)

// One weight of a launch.  The tensor maps live in the kernel's parameter space; a role passes the
// address of the map of the problem it is working on to the copy engine.
struct alignas(64) WgradProblem {
  CUtensorMap tm_dy, tm_x;       // operand panels: boxes of 64 columns x one stage of token rows
  CUtensorMap tm_w, tm_m, tm_v;  // boxes of 128 rows x one swizzle row of a chunk, for the loads and the stores
  int BT, V, H;
  int num_kb;          // ceil(BT / BK)
  int tiles_m;         // row tiles of TILE_M * CG rows
  int tiles_n;         // column tiles of TILE_N columns
  int unit_base;       // number of this problem's first unit in the launch
  int split_from;      // units (counted from unit_base) below this are whole tiles; the rest are 128-column halves of the following tiles
  int num_units;
  int ld_scale;        // row pitch of the scale arrays, in floats
  const uint8_t* dy;   // bf16 operands as the tensor maps see them (for the start-up L2 prefetch)
  const uint8_t* x;
  long long ld_dy_bytes, ld_x_bytes;
  float* m_scale;      // int8 / fp8-block: (V, H/64) row-major; fp8-tensor: one scalar
  float* v_scale;
  float* m_absmax;     // fp8-tensor: next-step absmax accumulators (atomic max)
  float* v_absmax;
  const Hyper* hyper_dev;  // optional: hyper-parameters read from device memory instead of `hyper`
  Hyper hyper;
};

struct WgradGroup {
  int n;               // problems in this launch
  int num_units;       // = clusters in the grid
  int* status;         // device status word: 0 = ok
  WgradProblem prob[MAX_GROUP];
};

// bytes one pipeline stage of W + moments takes for a chunk of `cn` columns
__host__ __device__ constexpr int state_stage_bytes(int wes, int ses, int nmom, int cn) {
  return 128 * cn * (wes + nmom * ses);
}

// CG = 1: one CTA per 128 x 256 tile.  CG = 2: a pair of CTAs (cluster of two, tcgen05 cta_group::2)
// per 256 x 256 tile; each CTA owns 128 rows and stages only HALF of the X panel (the pair MMA reads
// both halves), which cuts the L2 -> SM panel traffic per output by a third.
template <int W_DT, int ST, int OPT, int CG = 1>
struct WgradCfg {
  static constexpr int kWES = (W_DT == DT_BF16) ? 2 : 4;
  static constexpr int kNMom = num_moments(OPT);
  static constexpr int kSES = state_elem_size(ST);
  // Epilogue warps: eight (two groups of four, one accumulator row per thread).  With
  // FORGE_WIDE_EPILOGUE the block-quantised modes take sixteen (two groups of eight): TWO lanes of a
  // warp then share a row (tcgen05.ld shape 16x32bx2), 32 columns of the 64-column quantisation block
  // each, the block absmax is agreed by one shuffle, a thread carries half the values and every
  // scheduler has four epilogue warps.  It gives the same bits and is kept as a measured experiment:
  // at the 96 registers that 640 threads leave it spills, executes 24 % more instructions, and the
  // issue rate stays at 0.42 per scheduler and cycle as with eight warps, so it is slower.
  static constexpr bool kWide = FORGE_WIDE_EPILOGUE && (ST == ST_INT8 || ST == ST_FP8_BLOCK) && (W_DT == DT_BF16);
  static constexpr int kEpiWarps = kWide ? 16 : 8;
  static constexpr int kThreads = (EPI_WARP0 + kEpiWarps) * 32;
  // Token rows per operand stage.  With at most one moment (SGD, momentum, Lion) the state stream
  // is short and the kernel is bound by the panel loads; what limits those is the number of copy
  // operations one thread can issue (four per stage), so these optimizers take 64 rows per stage:
  // 14336 x 4096 plain SGD 89 -> 66 us.  With two moments the deeper state ring that 32-row
  // stages leave room for matters more (AdamW bf16 with 64-row stages: 132 -> 142 us).
  static constexpr int kBK = (kNMom < 2) ? 2 * OP_BK : OP_BK;
  static constexpr int kBaseStagesWanted = (kNMom < 2) ? ((CG == 2) ? 3 : 2) : ((CG == 2) ? OP_STAGES + 2 : OP_STAGES);
  static constexpr int kBaseStages = kBaseStagesWanted > 0 ? kBaseStagesWanted : 1;
  static constexpr int kOpStageBytes = (TILE_M + TILE_N / CG) * kBK * 2;
  static constexpr int kCtrlBytes = 1024;
  static constexpr int kRoom = SMEM_BUDGET - kCtrlBytes - 1024 - kBaseStages * kOpStageBytes;
  // 64-column chunks when four such stages fit (always with one-byte codes, whose quantisation block
  // is 64 columns); otherwise 32-column chunks, which buy a deeper ring for the same bytes
#ifdef FORGE_FORCE_CN32
  static constexpr int kCN = (kSES == 1) ? 64 : 32;
#else
  static constexpr int kCN = (kSES == 1 || 4 * state_stage_bytes(kWES, kSES, kNMom, 64) <= kRoom) ? 64 : 32;
#endif
  static constexpr int kNumChunks = TILE_N / kCN;
  static constexpr int kWRB = kCN * kWES;                      // bytes per W row inside a chunk
  static constexpr int kSRB = (kNMom > 0) ? kCN * kSES : 0;    // bytes per moment row inside a chunk
  static constexpr int kWBytes = 128 * kWRB;
  static constexpr int kSBytes = 128 * kSRB;
  static constexpr int kStageBytes = kWBytes + kNMom * kSBytes;
  static constexpr int kNSS_raw = kRoom / kStageBytes;
  static constexpr int kNSS_cap = kNSS_raw >= 8 ? 8 : (kNSS_raw >= 6 ? 6 : (kNSS_raw >= 4 ? 4 : 2));   // even, see the file comment
  static constexpr int kNSS = kNSS_cap > FORGE_MAX_STATE_STAGES ? FORGE_MAX_STATE_STAGES : kNSS_cap;
  // Shared memory the state ring leaves over goes to operand stages (at most eight): with small
  // states (plain SGD, one moment) the kernel is bound by the panel loads, whose rate is the bytes
  // in flight over the L2 latency.
  static constexpr int kSpare = kRoom - kNSS * kStageBytes;
  static constexpr int kExtraStages = (kSpare / kOpStageBytes < 8 - kBaseStages) ? kSpare / kOpStageBytes : 8 - kBaseStages;
#ifdef FORGE_NO_EXTRA_OP
  static constexpr int kNStage = kBaseStages;
#else
  static constexpr int kNStage = kBaseStages + (kExtraStages > 0 ? kExtraStages : 0);
#endif
  static constexpr int kSmemBytes = kCtrlBytes + 1024 + kNStage * kOpStageBytes + kNSS * kStageBytes;
  static_assert(kNSS_raw >= 2, "two state stages must fit in shared memory");
  static_assert(kSES != 1 || kCN == 64, "one-byte codes need 64-column chunks (the quantisation block)");
};

constexpr int TQ_SLOTS = 4;

struct alignas(16) CtrlBlock {
  uint64_t op_full[8];
  uint64_t op_empty[8];
  uint64_t st_full[8];
  uint64_t st_empty[8];
  uint64_t st_done[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t tq_full[TQ_SLOTS];    // unit queue: filled by the scheduler (st.async, 4 bytes each)
  uint64_t tq_empty[TQ_SLOTS];   // ... and drained by every other role of the cluster (leader CTA's copy is used)
  uint64_t clc_bar;              // completion of a cluster-launch-control request
  uint64_t fill_gate;            // operand producer -> state producer: the first unit's panel loads are all queued
  uint4 clc_resp;                // its 16-byte answer
  int tq_unit[TQ_SLOTS];
  uint32_t tmem_base;
  int abort_word;
};
static_assert(sizeof(CtrlBlock) <= 1024, "control block must fit in its reserved kilobyte");

// roles other than the scheduler that read the unit queue, per CTA: MMA issuer (leader) or operand
// producer (second CTA of a pair), state producer, store issuer, the epilogue warps

// ------------------------------------------------------------------------------------------------
template <int W_DT, int ST, int OPT, int CG>
__global__ void __launch_bounds__((WgradCfg<W_DT, ST, OPT, CG>::kThreads), 1)
forge_wgrad_kernel(const __grid_constant__ WgradGroup gp) {
  using Cfg = WgradCfg<W_DT, ST, OPT, CG>;
  constexpr int BK = Cfg::kBK;
  constexpr int NSTAGE = Cfg::kNStage;
  constexpr int NSS = Cfg::kNSS;
  constexpr int WES = Cfg::kWES;
  constexpr int SES = Cfg::kSES;
  constexpr int NMOM = Cfg::kNMom;
  constexpr int CN = Cfg::kCN;                 // columns per chunk
  constexpr int NG = CN / 16;                  // 16-column groups per chunk
  constexpr int WRB = Cfg::kWRB;
  constexpr int SRB = Cfg::kSRB;
  constexpr int WBC = BoxGeom<WRB>::kBoxRowBytes / WES;                 // columns per W box
  constexpr int SBC = (NMOM > 0) ? BoxGeom<SRB>::kBoxRowBytes / (SES > 0 ? SES : 1) : 1;
  constexpr bool WIDE = Cfg::kWide;
  constexpr int NUM_EPI_WARPS = Cfg::kEpiWarps;
  constexpr int GROUP_WARPS = NUM_EPI_WARPS / 2;          // warps that update one chunk together
  constexpr int TQ_READERS_PER_CTA = 3 + NUM_EPI_WARPS;
  constexpr int A_BYTES = TILE_M * BK * 2;
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

  // pair mode: rank 0 of the cluster is the leader (issues the MMAs, owns op_full and acc_empty)
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int first_unit = static_cast<int>(cluster_id_x());   // == blockIdx.x / CG

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&ctrl->op_full[i], 1); mbar_init(&ctrl->op_empty[i], 1); }
    for (int i = 0; i < NSS; ++i) {
      mbar_init(&ctrl->st_full[i], 1);
      mbar_init(&ctrl->st_empty[i], 1);
      mbar_init(&ctrl->st_done[i], GROUP_WARPS);   // one arrival per warp of the group that updated the chunk
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&ctrl->acc_full[i], 1); mbar_init(&ctrl->acc_empty[i], NUM_EPI_WARPS * CG); }
    for (int i = 0; i < TQ_SLOTS; ++i) { mbar_init(&ctrl->tq_full[i], 1); mbar_init(&ctrl->tq_empty[i], TQ_READERS_PER_CTA * CG); }
    mbar_init(&ctrl->clc_bar, 1);
    mbar_init(&ctrl->fill_gate, 1);
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
  // Problem a unit belongs to.  Units are numbered problem after problem; a launch has at most
  // MAX_GROUP problems, so a short scan does.
  auto locate = [&](int unit) -> const WgradProblem* {
    int i = 0;
    while (i + 1 < gp.n && unit >= gp.prob[i + 1].unit_base) ++i;
    return &gp.prob[i];
  };
  {
    const WgradProblem* p0 = locate(first_unit);
    if (warp == 0 && lane == 0) { prefetch_tmap(&p0->tm_dy); prefetch_tmap(&p0->tm_x); }
    if (warp == 2 && lane == 0) {
      prefetch_tmap(&p0->tm_w);
      if (NMOM > 0) prefetch_tmap(&p0->tm_m);
      if (NMOM > 1) prefetch_tmap(&p0->tm_v);
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  // unit number -> problem, row tile, first column, width (TILE_N, or TILE_N / 2 for a half)
  const WgradProblem* pp = nullptr;
  auto decode_unit = [&](int unit, int& row_tile, int& col0, int& ncols) {
    pp = locate(unit);
    const int u = unit - pp->unit_base;
    int tile = u, half = 0;
    ncols = TILE_N;
    if (u >= pp->split_from) {
      tile = pp->split_from + ((u - pp->split_from) >> 1);
      half = (u - pp->split_from) & 1;
      ncols = TILE_N / 2;
    }
    row_tile = tile / pp->tiles_n;
    col0 = (tile - row_tile * pp->tiles_n) * TILE_N + half * (TILE_N / 2);
  };
  // the leader CTA's tq_empty[0], where every reader of the cluster reports that it has taken a unit
  const uint32_t tq_empty0 = (CG == 2) ? map_to_cta(smem_u32(&ctrl->tq_empty[0]), 0) : smem_u32(&ctrl->tq_empty[0]);
  // Take the next unit from the queue (one thread of a role).  Negative: no more work, or a wait gave up.
  uint32_t tq_pos = 0;
  auto pop_unit = [&]() -> int {
    const uint32_t slot = tq_pos % TQ_SLOTS;
    if (!mbar_wait(&ctrl->tq_full[slot], (tq_pos / TQ_SLOTS) & 1, abort_word, ERR_WAIT_TQ_FULL)) return -1;
    const int unit = *reinterpret_cast<volatile int*>(&ctrl->tq_unit[slot]);
    if constexpr (CG == 2) mbar_arrive_cluster(tq_empty0 + slot * 8);
    else mbar_arrive(&ctrl->tq_empty[slot]);
    ++tq_pos;
    return unit;
  };
  int row_tile, col0, ncols;

  if (warp == 0) {
    // ------------------------------------------------------------------ operand producer
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();
      uint32_t it = 0;
      // the scheduler (leader) starts with the unit of its own cluster and has the next request in flight
      int unit = first_unit;
      bool more = true;        // the last request was answered with a unit
      uint32_t req = 0;        // requests answered so far
      bool gate_open = false;  // the state producer has been told that the first unit's loads are queued
      if (cta_rank == 0) {
        mbar_expect_tx(&ctrl->clc_bar, 16);
        clc_try_cancel(&ctrl->clc_resp, &ctrl->clc_bar);
      }
      for (;;) {
        if (cta_rank == 0) {
          // publish `unit` (negative: the end) to the other roles of both CTAs
          const uint32_t slot = tq_pos % TQ_SLOTS;
          if (!mbar_wait(&ctrl->tq_empty[slot], ((tq_pos / TQ_SLOTS) & 1) ^ 1, abort_word, ERR_WAIT_TQ_EMPTY)) goto done;
#pragma unroll
          for (uint32_t rk = 0; rk < static_cast<uint32_t>(CG); ++rk) {
            const uint32_t bar = (CG == 2) ? map_to_cta(smem_u32(&ctrl->tq_full[slot]), rk) : smem_u32(&ctrl->tq_full[slot]);
            const uint32_t dst = (CG == 2) ? map_to_cta(smem_u32(&ctrl->tq_unit[slot]), rk) : smem_u32(&ctrl->tq_unit[slot]);
            mbar_expect_tx_cluster(bar, 4);
            st_async_u32(dst, static_cast<uint32_t>(unit), bar);
          }
          ++tq_pos;
        } else {
          unit = pop_unit();
        }
        if (unit < 0) break;
        decode_unit(unit, row_tile, col0, ncols);
        const int row0 = row_tile * (TILE_M * CG) + static_cast<int>(cta_rank) * TILE_M;
        const int b_cols = ncols / CG;             // columns of the X panel this CTA stages
        const uint32_t b_bytes = static_cast<uint32_t>(b_cols) * BK * 2;
        const int num_kb = pp->num_kb;
        const CUtensorMap* tm_dy = &pp->tm_dy;
        const CUtensorMap* tm_x = &pp->tm_x;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          if (!mbar_wait(&ctrl->op_empty[s], ph ^ 1, abort_word, ERR_WAIT_OP_EMPTY)) goto done;
          uint8_t* a = op_buf + s * Cfg::kOpStageBytes;
          uint8_t* b = a + A_BYTES;
          if constexpr (CG == 2) {
            // both CTAs' copies count on the LEADER's barrier; the leader expects the bytes of both
            const uint32_t full_leader = map_to_cta(smem_u32(&ctrl->op_full[s]), 0);
            if (cta_rank == 0) mbar_expect_tx(&ctrl->op_full[s], 2 * (A_BYTES + b_bytes));
            const int bcol0 = col0 + static_cast<int>(cta_rank) * b_cols;
#pragma unroll
            for (int i = 0; i < TILE_M / 64; ++i)
              tma_load_2d_pair(a + i * SLAB_BYTES, tm_dy, full_leader, row0 + 64 * i, kb * BK, pol);
            for (int i = 0; i < b_cols / 64; ++i)
              tma_load_2d_pair(b + i * SLAB_BYTES, tm_x, full_leader, bcol0 + 64 * i, kb * BK, pol);
          } else {
            mbar_expect_tx(&ctrl->op_full[s], A_BYTES + b_bytes);
#pragma unroll
            for (int i = 0; i < TILE_M / 64; ++i)
              tma_load_2d(a + i * SLAB_BYTES, tm_dy, &ctrl->op_full[s], row0 + 64 * i, kb * BK, pol);
            for (int i = 0; i < b_cols / 64; ++i)
              tma_load_2d(b + i * SLAB_BYTES, tm_x, &ctrl->op_full[s], col0 + 64 * i, kb * BK, pol);
          }
        }
        if (!gate_open) { mbar_arrive(&ctrl->fill_gate); gate_open = true; }   // end of the first unit
        if (cta_rank == 0) {
          // the answer to the request made one unit ago has had a whole tile's loads to arrive
          if (more) {
            if (!mbar_wait(&ctrl->clc_bar, req & 1, abort_word, ERR_WAIT_CLC)) goto done;
            ++req;
            uint32_t first_cta = 0;
            more = clc_query(&ctrl->clc_resp, first_cta);
            unit = more ? static_cast<int>(first_cta / CG) : -1;
            if (more) {
              mbar_expect_tx(&ctrl->clc_bar, 16);
              clc_try_cancel(&ctrl->clc_resp, &ctrl->clc_bar);
            }
          } else {
            unit = -1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc0 = make_idesc_bf16(TILE_M * CG, 0, true, true);
      uint32_t it = 0;
      uint32_t tile_it = 0;
      for (int unit; (unit = pop_unit()) >= 0; ++tile_it) {
        decode_unit(unit, row_tile, col0, ncols);
        const uint32_t idesc = idesc0 | (static_cast<uint32_t>(ncols >> 3) << 17);   // N field
        const int buf = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&ctrl->acc_empty[buf], aph ^ 1, abort_word, ERR_WAIT_ACC_EMPTY)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * TILE_N;
        const int num_kb = pp->num_kb;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
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
            if constexpr (CG == 2) umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // frees the stage in both CTAs of a pair
          if constexpr (CG == 2) umma_commit_pair(&ctrl->op_empty[s], 3);
          else umma_commit(&ctrl->op_empty[s]);
        }
        if constexpr (CG == 2) umma_commit_pair(&ctrl->acc_full[buf], 3);
        else umma_commit(&ctrl->acc_full[buf]);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ state producer
    if (lane == 0) {
      // Normal priority, not evict-first: a chunk row is only 64-128 bytes, the L2 fetches 256-byte
      // granules, and the rest of each granule is wanted by the next chunks a few microseconds
      // later.  With evict-first those lines were dropped and fetched again (measured: 158 us ->
      // 126 us on a 14336 x 4096 bf16 update when this policy was changed).
      const uint64_t pol = policy_evict_normal();
      uint32_t q = 0;
      for (int unit; (unit = pop_unit()) >= 0;) {
        decode_unit(unit, row_tile, col0, ncols);
        const int row0 = row_tile * (TILE_M * CG) + static_cast<int>(cta_rank) * TILE_M;
        const int nch = ncols / CN;
        const CUtensorMap* tm_w = &pp->tm_w;
        const CUtensorMap* tm_m = &pp->tm_m;
        const CUtensorMap* tm_v = &pp->tm_v;
        if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
          // The epilogue threads read their rows' block scales straight from global memory at the top
          // of a tile; this thread knows the tile several microseconds earlier and pulls the lines
          // into L2 (one 16-byte group of scales per row, tensor and tile).
          for (int rr = 0; rr < TILE_M; ++rr) {
            if (row0 + rr < pp->V) {
              const size_t off = static_cast<size_t>(row0 + rr) * pp->ld_scale + (col0 >> 6);
              prefetch_l2(pp->m_scale + off);
              prefetch_l2(pp->v_scale + off);
            }
          }
        }
        for (int c = 0; c < nch; ++c, ++q) {
          const int s = q % NSS;
          const uint32_t ph = (q / NSS) & 1;
          if (!mbar_wait(&ctrl->st_empty[s], ph ^ 1, abort_word, ERR_WAIT_ST_EMPTY)) goto done;
          // Start-up: the copy engine serves requests in order and everything is cold, so a full ring
          // of state loads ahead of the first tile's panels doubles the time to the first accumulator
          // (8 us instead of 4).  Two chunks are enough for the epilogue to start on; the rest wait
          // until the producer has queued the whole first panel.
          if (q == FORGE_FILL_GATE_CHUNKS) {
            if (!mbar_wait(&ctrl->fill_gate, 0, abort_word, ERR_WAIT_FILL_GATE)) goto done;
          }
          uint8_t* wb = st_buf + s * Cfg::kStageBytes;
          mbar_expect_tx(&ctrl->st_full[s], Cfg::kStageBytes);
          const int cc = col0 + c * CN;
#pragma unroll
          for (int bx = 0; bx < BoxGeom<WRB>::kBoxes; ++bx)
            tma_load_2d(wb + bx * BoxGeom<WRB>::kBoxBytes, tm_w, &ctrl->st_full[s], cc + bx * WBC, row0, pol);
          if constexpr (NMOM > 0) {
            uint8_t* mb = wb + Cfg::kWBytes;
#pragma unroll
            for (int bx = 0; bx < BoxGeom<SRB>::kBoxes; ++bx)
              tma_load_2d(mb + bx * BoxGeom<SRB>::kBoxBytes, tm_m, &ctrl->st_full[s], cc + bx * SBC, row0, pol);
          }
          if constexpr (NMOM > 1) {
            uint8_t* vb = wb + Cfg::kWBytes + Cfg::kSBytes;
#pragma unroll
            for (int bx = 0; bx < BoxGeom<SRB>::kBoxes; ++bx)
              tma_load_2d(vb + bx * BoxGeom<SRB>::kBoxBytes, tm_v, &ctrl->st_full[s], cc + bx * SBC, row0, pol);
          }
        }
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ store issuer
    if (lane == 0) {
      // normal priority, so that the partial lines of neighbouring chunks merge in L2
      const uint64_t pol = policy_evict_normal();
      uint32_t q = 0;
      for (int unit; (unit = pop_unit()) >= 0;) {
        decode_unit(unit, row_tile, col0, ncols);
        const int row0 = row_tile * (TILE_M * CG) + static_cast<int>(cta_rank) * TILE_M;
        const int nch = ncols / CN;
        const CUtensorMap* tm_w = &pp->tm_w;
        const CUtensorMap* tm_m = &pp->tm_m;
        const CUtensorMap* tm_v = &pp->tm_v;
        const int pV = pp->V, pH = pp->H;
        for (int c = 0; c < nch; ++c, ++q) {
          const int s = q % NSS;
          const uint32_t ph = (q / NSS) & 1;
          // the four warps that updated this chunk made their writes visible to the async proxy
          // (fence.proxy.async) before arriving
          if (!mbar_wait(&ctrl->st_done[s], ph, abort_word, ERR_WAIT_ST_DONE)) goto done;
          uint8_t* wb = st_buf + s * Cfg::kStageBytes;
          const int cc = col0 + c * CN;
          if (row0 < pV && cc < pH) {   // rows / columns past the edge of a started box are clipped
#pragma unroll
            for (int bx = 0; bx < BoxGeom<WRB>::kBoxes; ++bx)
              if (cc + bx * WBC < pH) tma_store_2d(tm_w, wb + bx * BoxGeom<WRB>::kBoxBytes, cc + bx * WBC, row0, pol);
            if constexpr (NMOM > 0) {
              uint8_t* mb = wb + Cfg::kWBytes;
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SRB>::kBoxes; ++bx)
                if (cc + bx * SBC < pH) tma_store_2d(tm_m, mb + bx * BoxGeom<SRB>::kBoxBytes, cc + bx * SBC, row0, pol);
            }
            if constexpr (NMOM > 1) {
              uint8_t* vb = wb + Cfg::kWBytes + Cfg::kSBytes;
#pragma unroll
              for (int bx = 0; bx < BoxGeom<SRB>::kBoxes; ++bx)
                if (cc + bx * SBC < pH) tma_store_2d(tm_v, vb + bx * BoxGeom<SRB>::kBoxBytes, cc + bx * SBC, row0, pol);
            }
          }
          tma_store_commit();
          // the stage goes back to the producer as soon as the copy engine has read it
          tma_store_wait_read<0>();
          mbar_arrive(&ctrl->st_empty[s]);
        }
      }
      tma_store_wait_all<0>();
    }
  } else if (warp >= EPI_WARP0) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int wg = (warp - EPI_WARP0) / GROUP_WARPS;       // 0 or 1: the chunks this warp's group takes
    // row inside the tile, and -- wide form -- which 32 columns of the chunk this lane has
    const int hh = WIDE ? (((warp - EPI_WARP0) % GROUP_WARPS) >> 2) : 0;      // 16-row half of the quarter
    const int ch = WIDE ? (lane >> 4) : 0;
    const int r = WIDE ? (quarter * 32 + hh * 16 + (lane & 15)) : (quarter * 32 + lane);
    const uint32_t tmem_lane = static_cast<uint32_t>(WIDE ? (quarter * 32 + hh * 16) : (quarter * 32)) << 16;
    // per-problem values, (re)loaded when the unit at hand belongs to another problem than the last
    const WgradProblem* cur = nullptr;
    Hyper hy = gp.prob[0].hyper;
    float s_m_t = 1.0f, s_v_t = 1.0f, inv_m_t = 1.0f, inv_v_t = 1.0f;
    float amax_m_t = 0.0f, amax_v_t = 0.0f;
    // fp8 per tensor: this warp's running maxima of |m'| and |v'| go to the problem's accumulators
    auto flush_absmax = [&](const WgradProblem* q) {
      if constexpr (ST == ST_FP8_TENSOR) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          amax_m_t = fmaxf(amax_m_t, __shfl_xor_sync(0xffffffffu, amax_m_t, o));
          amax_v_t = fmaxf(amax_v_t, __shfl_xor_sync(0xffffffffu, amax_v_t, o));
        }
        if (lane == 0) {
          // non-negative floats order like their bit patterns
          atomicMax(reinterpret_cast<unsigned int*>(q->m_absmax), __float_as_uint(amax_m_t));
          atomicMax(reinterpret_cast<unsigned int*>(q->v_absmax), __float_as_uint(amax_v_t));
        }
        amax_m_t = 0.0f;
        amax_v_t = 0.0f;
      }
    };
    uint32_t tile_it = 0;
    uint32_t q_base = 0;   // chunks of the tiles before this one (always even)
    bool ok = true;
    // Start-up: nothing to update until the first accumulator is complete, and its panels are cold
    // in L2.  With five operand stages the producer can only have five token blocks in flight, so
    // the first tile would take three to four DRAM round trips; these 256 idle threads ask L2 for
    // the whole panel of the first unit at once instead (the unit of a cluster's own index is known
    // without the queue).
    decode_unit(first_unit, row_tile, col0, ncols);
    if (pp->num_kb > 0) {
      const int a_col0 = row_tile * (TILE_M * CG) + static_cast<int>(cta_rank) * TILE_M;
      const int b_cols = ncols / CG;
      const int b_col0 = col0 + static_cast<int>(cta_rank) * ((CG == 2) ? b_cols : 0);
      const int lines_a = TILE_M / 64, per_row = lines_a + b_cols / 64;   // 128-byte lines per token row
      const int rows = pp->BT < 1024 ? pp->BT : 1024;
      for (int idx = static_cast<int>(threadIdx.x) - EPI_WARP0 * 32; idx < rows * per_row; idx += NUM_EPI_WARPS * 32) {
        const int row = idx / per_row, l = idx - row * per_row;
        if (l < lines_a) {
          const int col = a_col0 + 64 * l;
          if (col < pp->V) prefetch_l2(pp->dy + row * pp->ld_dy_bytes + col * 2);
        } else {
          const int col = b_col0 + 64 * (l - lines_a);
          if (col < pp->H) prefetch_l2(pp->x + row * pp->ld_x_bytes + col * 2);
        }
      }
    }
    for (; ok; ++tile_it) {
      // every lane waits for the unit and reads it; one lane reports that the warp has it
      const uint32_t slot = tq_pos % TQ_SLOTS;
      ok = mbar_wait(&ctrl->tq_full[slot], (tq_pos / TQ_SLOTS) & 1, abort_word, ERR_WAIT_TQ_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int unit = *reinterpret_cast<volatile int*>(&ctrl->tq_unit[slot]);
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2) mbar_arrive_cluster(tq_empty0 + slot * 8);
        else mbar_arrive(&ctrl->tq_empty[slot]);
      }
      ++tq_pos;
      if (unit < 0) break;
      decode_unit(unit, row_tile, col0, ncols);
      if (pp != cur) {
        if (cur != nullptr) flush_absmax(cur);
        cur = pp;
        hy = (pp->hyper_dev != nullptr) ? *pp->hyper_dev : pp->hyper;
        if constexpr (ST == ST_FP8_TENSOR) {
          s_m_t = *pp->m_scale;
          s_v_t = *pp->v_scale;
          inv_m_t = f_div(1.0f, s_m_t);
          inv_v_t = f_div(1.0f, s_v_t);
        }
      }
      const int pV = pp->V, pH = pp->H;
      const int row0 = row_tile * (TILE_M * CG) + static_cast<int>(cta_rank) * TILE_M;
      const int half_chunks = ncols / (2 * CN);   // chunks of this tile per epilogue group
      const int buf = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const int grow = row0 + r;

      // per-(row, 64-column block) scales of this thread's two chunks
      float sc_m[2] = {1.0f, 1.0f}, sc_v[2] = {1.0f, 1.0f};
      if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int cb = (col0 >> 6) + wg + 2 * i;
          if (grow < pV && cb * 64 < pH) {
            sc_m[i] = __ldg(pp->m_scale + static_cast<size_t>(grow) * pp->ld_scale + cb);
            sc_v[i] = __ldg(pp->v_scale + static_cast<size_t>(grow) * pp->ld_scale + cb);
          }
        }
      }

      ok = mbar_wait(&ctrl->acc_full[buf], aph, abort_word, ERR_WAIT_ACC_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

#pragma unroll 1
      for (int i = 0; i < half_chunks; ++i) {
        const int c = wg + 2 * i;
        const uint32_t q = q_base + c;
        const int s = q % NSS;
        const uint32_t ph = (q / NSS) & 1;

        // accumulator row: the CN fp32 columns of this chunk.  The block-quantised modes fetch it in
        // groups of 16 columns as they go (they keep 64 new second moments in registers already)
        constexpr bool kTmemScratch = (ST == ST_INT8 || ST == ST_FP8_BLOCK);
        constexpr int ACC_REGS = kTmemScratch ? 16 : CN;
        uint32_t acc[ACC_REGS];
        const uint32_t acc_taddr = tmem_base + tmem_lane + static_cast<uint32_t>(buf * TILE_N + c * CN);
        if constexpr (WIDE) {
          tmem_ld_16x16_split32(acc_taddr, &acc[0]);
        } else if constexpr (kTmemScratch) {
          tmem_ld_32x16(acc_taddr, &acc[0]);
        } else {
          tmem_ld_32x32(acc_taddr, &acc[0]);
          if constexpr (CN == 64) tmem_ld_32x32(acc_taddr + 32, &acc[32]);
        }
        ok = mbar_wait(&ctrl->st_full[s], ph, abort_word, ERR_WAIT_ST_FULL);
        ok = __all_sync(0xffffffffu, ok);
        tmem_ld_wait();
        if (!ok) break;
        if (!kTmemScratch && i == half_chunks - 1) {
          // this warp's last read of the accumulator: hand the buffer back to the MMA issuer now,
          // not after the update of the chunk
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->acc_empty[buf]), 0));
            else mbar_arrive(&ctrl->acc_empty[buf]);
          }
        }
        const bool no_tokens = pp->num_kb == 0;
        if (no_tokens) {
#pragma unroll
          for (int k = 0; k < ACC_REGS; ++k) acc[k] = 0u;
        }

        uint8_t* wb = st_buf + s * Cfg::kStageBytes;
        uint8_t* mb = wb + Cfg::kWBytes;
        uint8_t* vb = mb + Cfg::kSBytes;

        if constexpr (OPT == OPT_SGD) {
          Raw16<WES> rw = load_raw<WES, WRB>(wb, r, 0);
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            Raw16<WES> nw;
            if (g + 1 < NG) nw = load_raw<WES, WRB>(wb, r, g + 1);
            float w[16];
            unpack16<WES>(rw, w);
#pragma unroll
            for (int k = 0; k < 16; ++k) w[k] = sgd_update(w[k], __uint_as_float(acc[16 * g + k]), hy);
            store_raw<WES, WRB>(wb, r, g, pack16<WES>(w));
            if (g + 1 < NG) rw = nw;
          }
        } else if constexpr (OPT == OPT_SGDM || OPT == OPT_LION) {
          Raw16<WES> rw = load_raw<WES, WRB>(wb, r, 0);
          Raw16<SES> rm = load_raw<SES, SRB>(mb, r, 0);
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            Raw16<WES> nw;
            Raw16<SES> nm;
            if (g + 1 < NG) {
              nw = load_raw<WES, WRB>(wb, r, g + 1);
              nm = load_raw<SES, SRB>(mb, r, g + 1);
            }
            float w[16], m[16];
            unpack16<WES>(rw, w);
            unpack16<SES>(rm, m);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float gr = __uint_as_float(acc[16 * g + k]);
              w[k] = (OPT == OPT_SGDM) ? sgdm_update(w[k], gr, m[k], hy) : lion_update(w[k], gr, m[k], hy);
            }
            store_raw<WES, WRB>(wb, r, g, pack16<WES>(w));
            store_raw<SES, SRB>(mb, r, g, pack16<SES>(m));
            if (g + 1 < NG) { rw = nw; rm = nm; }
          }
        } else if constexpr (ST == ST_F32 || ST == ST_BF16) {
          Raw16<WES> rw = load_raw<WES, WRB>(wb, r, 0);
          Raw16<SES> rm = load_raw<SES, SRB>(mb, r, 0);
          Raw16<SES> rv = load_raw<SES, SRB>(vb, r, 0);
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            Raw16<WES> nw;
            Raw16<SES> nm, nv;
            if (g + 1 < NG) {
              nw = load_raw<WES, WRB>(wb, r, g + 1);
              nm = load_raw<SES, SRB>(mb, r, g + 1);
              nv = load_raw<SES, SRB>(vb, r, g + 1);
            }
            float w[16], m[16], v[16];
            unpack16<WES>(rw, w);
            unpack16<SES>(rm, m);
            unpack16<SES>(rv, v);
#pragma unroll
            for (int k = 0; k < 16; k += 2) {
              float2 m2 = make_float2(m[k], m[k + 1]), v2 = make_float2(v[k], v[k + 1]);
              const float2 w2 = adamw_update2(make_float2(w[k], w[k + 1]),
                                              make_float2(__uint_as_float(acc[16 * g + k]), __uint_as_float(acc[16 * g + k + 1])),
                                              m2, v2, hy);
              w[k] = w2.x; w[k + 1] = w2.y;
              m[k] = m2.x; m[k + 1] = m2.y;
              v[k] = v2.x; v[k + 1] = v2.y;
            }
            store_raw<WES, WRB>(wb, r, g, pack16<WES>(w));
            store_raw<SES, SRB>(mb, r, g, pack16<SES>(m));
            store_raw<SES, SRB>(vb, r, g, pack16<SES>(v));
            if (g + 1 < NG) { rw = nw; rm = nm; rv = nv; }
          }
        } else if constexpr (ST == ST_INT8 || ST == ST_FP8_BLOCK) {
          // The 64-column quantisation block is this thread's whole chunk row -- or, in the wide form,
          // the row of two lanes of this warp (lane and lane ^ 16), 32 columns each.  Pass 1 dequantises,
          // updates W and tracks the block absmax; the new second moments stay in registers, the new
          // first moments are parked in the accumulator's own tensor-memory columns, which this thread
          // has already read (holding both in registers spilled).  Pass 2 requantises them with the
          // new scale.  No recomputation; one shuffle per block in the wide form, none otherwise.
          constexpr int MYG = WIDE ? 2 : NG;            // 16-column groups per thread
          const int g0 = WIDE ? 2 * ch : 0;             // this thread's first group inside the chunk row
          const float sm_old = (i == 0) ? sc_m[0] : sc_m[1];
          const float sv_old = (i == 0) ? sc_v[0] : sc_v[1];
          const float2 sm_old2 = make_float2(sm_old, sm_old), sv_old2 = make_float2(sv_old, sv_old);
          const uint32_t scratch = acc_taddr;
          // 16 tensor-memory columns of group g (the wide form's split load adds the other lane's 32 itself)
          auto tm_ld = [&](int g, uint32_t* dst) {
            if constexpr (WIDE) tmem_ld_16x16_split32(scratch + 16 * g, dst);
            else tmem_ld_32x16(scratch + 16 * g, dst);
          };
          auto tm_st = [&](int g, const uint32_t* src) {
            if constexpr (WIDE) tmem_st_16x16_split32(scratch + 16 * g, src);
            else tmem_st_32x16(scratch + 16 * g, src);
          };
          float vv[16 * MYG];
          float am = 0.0f, av = 0.0f;
#pragma unroll
          for (int g = 0; g < MYG; ++g) {
            float w[16];
            uint32_t mq[4], vq[4], mnew[16], acc_next[16];
            // the accumulator columns of the next group are on their way while this one is worked on
            if (g + 1 < MYG) tm_ld(g + 1, acc_next);
            unpack16<WES>(load_raw<WES, WRB>(wb, r, g0 + g), w);
            ld16_bytes(mb, r, g0 + g, mq);
            ld16_bytes(vb, r, g0 + g, vq);
            if constexpr (ST == ST_INT8) {
              // first moments are signed: flip the sign bits so that a byte reads as code + 128; second
              // moments are never negative and are taken as they are
#pragma unroll
              for (int j = 0; j < 4; ++j) mq[j] ^= 0x80808080u;
            }
#pragma unroll
            for (int k = 0; k < 16; k += 2) {
              float2 m2, v2;
              if constexpr (ST == ST_INT8) {
                m2 = int8x2_to_float(mq[k >> 2], k & 3);
                v2 = uint8x2_to_float(vq[k >> 2], k & 3);
              } else {
                e4m3x2_to_float(mq[k >> 2] >> (8 * (k & 3)), m2.x, m2.y);
                e4m3x2_to_float(vq[k >> 2] >> (8 * (k & 3)), v2.x, v2.y);
              }
              m2 = fmul2(m2, sm_old2);
              v2 = fmul2(v2, sv_old2);
              v2.x = fmaxf(v2.x, 1e-8f);
              v2.y = fmaxf(v2.y, 1e-8f);
              const float2 w2 = adamw_update2(make_float2(w[k], w[k + 1]),
                                              make_float2(__uint_as_float(acc[k]), __uint_as_float(acc[k + 1])),
                                              m2, v2, hy);
              w[k] = w2.x;
              w[k + 1] = w2.y;
              mnew[k] = __float_as_uint(m2.x);
              mnew[k + 1] = __float_as_uint(m2.y);
              vv[16 * g + k] = v2.x;
              vv[16 * g + k + 1] = v2.y;
              am = fmax3(am, fabsf(m2.x), fabsf(m2.y));
              av = fmax3(av, v2.x, v2.y);          // second moments are sums of non-negative terms
            }
            tm_st(g, mnew);
            store_raw<WES, WRB>(wb, r, g0 + g, pack16<WES>(w));
            if (g + 1 < MYG) {
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 16; ++k) acc[k] = no_tokens ? 0u : acc_next[k];
            }
          }
          tmem_st_wait();
          if constexpr (WIDE) {
            // the other half of the block lives in lane ^ 16
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 16));
            av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 16));
          }
          const float sm_new = (ST == ST_INT8) ? int8_scale(am) : fp8blk_scale(am);
          const float sv_new = (ST == ST_INT8) ? int8_scale(av) : fp8blk_scale(av);
          const float rsm = f_rcp(sm_new), rsv = f_rcp(sv_new);
          const float2 nsm2 = make_float2(-sm_new, -sm_new), nsv2 = make_float2(-sv_new, -sv_new);
          const float2 rsm2 = make_float2(rsm, rsm), rsv2 = make_float2(rsv, rsv);
          uint32_t mcur[16];
          tm_ld(0, mcur);
#pragma unroll
          for (int g = 0; g < MYG; ++g) {
            uint32_t mo[4], vo[4], mnext[16];
            tmem_ld_wait();
            if (g + 1 < MYG) tm_ld(g + 1, mnext);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int k = 4 * j;
              const float2 qm01 = div2_by_rcp(make_float2(__uint_as_float(mcur[k]), __uint_as_float(mcur[k + 1])), nsm2, rsm2);
              const float2 qm23 = div2_by_rcp(make_float2(__uint_as_float(mcur[k + 2]), __uint_as_float(mcur[k + 3])), nsm2, rsm2);
              const float2 qv01 = div2_by_rcp(make_float2(vv[16 * g + k], vv[16 * g + k + 1]), nsv2, rsv2);
              const float2 qv23 = div2_by_rcp(make_float2(vv[16 * g + k + 2], vv[16 * g + k + 3]), nsv2, rsv2);
              if constexpr (ST == ST_INT8) {
                mo[j] = int8x4_pack(int8x2_round(qm01), int8x2_round(qm23));
                vo[j] = int8x4_pack(int8x2_round(qv01), int8x2_round(qv23));
              } else {
                // |x / scale| < 448.5 by construction of the scale, and the conversion saturates
                mo[j] = e4m3x2_code_bits(qm01.x, qm01.y) | (e4m3x2_code_bits(qm23.x, qm23.y) << 16);
                vo[j] = e4m3x2_code_bits(qv01.x, qv01.y) | (e4m3x2_code_bits(qv23.x, qv23.y) << 16);
              }
            }
            st16_bytes(mb, r, g0 + g, mo);
            st16_bytes(vb, r, g0 + g, vo);
            if (g + 1 < MYG) {
#pragma unroll
              for (int k = 0; k < 16; ++k) mcur[k] = mnext[k];
            }
          }
          if (i == half_chunks - 1) {
            // last use of this accumulator buffer (as scratch): hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&ctrl->acc_empty[buf]), 0));
              else mbar_arrive(&ctrl->acc_empty[buf]);
            }
          }
          {
            const int cb = (col0 >> 6) + c;
            if (ch == 0 && grow < pV && cb * 64 < pH) {
              pp->m_scale[static_cast<size_t>(grow) * pp->ld_scale + cb] = sm_new;
              pp->v_scale[static_cast<size_t>(grow) * pp->ld_scale + cb] = sv_new;
            }
          }
        } else {  // ST_FP8_TENSOR
#pragma unroll
          for (int g = 0; g < NG; ++g) {
            float w[16];
            uint32_t mq[4], vq[4], mo[4] = {0, 0, 0, 0}, vo[4] = {0, 0, 0, 0};
            unpack16<WES>(load_raw<WES, WRB>(wb, r, g), w);
            ld16_bytes(mb, r, g, mq);
            ld16_bytes(vb, r, g, vq);
#pragma unroll
            for (int k = 0; k < 16; k += 2) {
              float2 m2, v2;
              e4m3x2_to_float(mq[k >> 2] >> (8 * (k & 3)), m2.x, m2.y);
              e5m2x2_to_float(vq[k >> 2] >> (8 * (k & 3)), v2.x, v2.y);
              m2 = fmul2(m2, make_float2(s_m_t, s_m_t));
              v2 = fmul2(v2, make_float2(s_v_t, s_v_t));
              const float2 w2 = adamw_update2(make_float2(w[k], w[k + 1]),
                                              make_float2(__uint_as_float(acc[16 * g + k]), __uint_as_float(acc[16 * g + k + 1])),
                                              m2, v2, hy);
              w[k] = w2.x;
              w[k + 1] = w2.y;
              // rows / columns beyond the matrix hold zeros (zero-filled loads), so they never raise
              // the running maxima
              amax_m_t = fmaxf(amax_m_t, fmaxf(fabsf(m2.x), fabsf(m2.y)));
              amax_v_t = fmaxf(amax_v_t, fmaxf(fabsf(v2.x), fabsf(v2.y)));
              // the conversions saturate to +-448 / +-57344, which is the reference's clamp
              const float2 mc = fmul2(m2, make_float2(inv_m_t, inv_m_t));
              const float2 vc = fmul2(v2, make_float2(inv_v_t, inv_v_t));
              mo[k >> 2] |= e4m3x2_code_bits(mc.x, mc.y) << (8 * (k & 3));
              vo[k >> 2] |= e5m2x2_code_bits(vc.x, vc.y) << (8 * (k & 3));
            }
            store_raw<WES, WRB>(wb, r, g, pack16<WES>(w));
            st16_bytes(mb, r, g, mo);
            st16_bytes(vb, r, g, vo);
          }
        }

        // hand the updated rows of this warp to the store issuer
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctrl->st_done[s]);
      }
      if (!ok) break;
      q_base += 2 * half_chunks;
    }
    if (cur != nullptr) flush_absmax(cur);
  }

done:
  // the single-lane roles leave their loops alone; bring every warp back together before the
  // CTA-wide barrier (an aligned barrier executed by a diverged warp is undefined)
  __syncwarp();
  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // error path: give copies in flight a bounded time to land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) __nanosleep(1000);
    if (threadIdx.x == 0 && gp.status != nullptr) atomicCAS(gp.status, 0, *abort_word);
    __syncthreads();
  }
  // a pair leaves together: the peer's shared memory and barriers stay valid until both are done
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace forge
