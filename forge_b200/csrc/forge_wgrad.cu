// C-ABI entry of the fused weight-gradient + optimizer update: validation, tensor maps, dispatch.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <vector>

#include "forge_host.h"
#include "forge_wgrad_kernel.cuh"

namespace forge {

// fp32 operands are split into bf16 high and low parts, x = hi + lo with hi = bf16(x) and
// lo = bf16(x - hi), and the product dY^T X is expanded as hi.hi + hi.lo + lo.hi by stacking three
// copies along the token axis (rows padded to a multiple of 64 with zeros):
//   A' = [dY_hi; dY_hi; dY_lo]   B' = [X_hi; X_lo; X_hi]
// so the same bf16 kernel runs with 3x the reduction length.  The dropped lo.lo term is below
// 2^-16 relative, i.e. tighter than the TF32 dot the reference uses for fp32 inputs.
__global__ void split_f32_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t ld,
                                 int64_t rows_pad, __nv_bfloat16* __restrict__ dst, int second_is_lo) {
  const int64_t n = rows_pad * cols;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / cols, c = i % cols;
    float x = 0.0f;
    if (r < rows) x = src[r * ld + c];
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    const __nv_bfloat16 lo = __float2bfloat16_rn(x - __bfloat162float(hi));
    dst[i] = hi;
    dst[n + i] = second_is_lo ? lo : hi;
    dst[2 * n + i] = second_is_lo ? hi : lo;
  }
}

// One validated problem of a launch: what the launcher needs to build the tensor maps and the
// kernel's per-problem parameters for whichever kernel configuration is chosen.
struct Prepared {
  void* W;
  void* m;
  void* v;
  int64_t V, H, ld_w, ld_state;
  // bf16 operands as the kernel reads them (the split copies for fp32 inputs); bt = token rows
  const void* dy;
  const void* x;
  int64_t bt, ld_dy, ld_x;
  float* m_scale;
  float* v_scale;
  int64_t ld_scale;
  float* m_absmax;
  float* v_absmax;
  Hyper hyper;
  const Hyper* hyper_dev;
  int32_t* status;
  int w_dtype, opt, st;
};

// Number of final tiles issued as 128-column halves when a launch has at least two rounds of
// tiles: by default one half per worker (measured on 14336 x 4096 and 4096 x 4096: 1.5 % and 3.7 %
// faster than whole tiles to the end; more halves were slower).  FORGE_TAIL_HALVES=<n> in the
// environment (a tuning aid, read once) overrides it.
static int64_t tail_halves(int64_t tiles, int64_t workers) {
  static const int env = [] {
    const char* e = getenv("FORGE_TAIL_HALVES");
    return e != nullptr ? atoi(e) : -1;
  }();
  if (env >= 0) return env;
  return tiles >= 2 * workers ? workers / 2 : 0;
}

// one launch for `n` problems (1 <= n <= MAX_GROUP) of one kernel configuration
template <int W_DT, int ST, int OPT, int CG>
static int launch_wgrad(const Prepared* items, int n, int sm_count, cudaStream_t stream) {
  using Cfg = WgradCfg<W_DT, ST, OPT, CG>;
  using WG = BoxGeom<Cfg::kWRB>;
  WgradGroup g;   // the kernel's parameter block (several kilobytes, passed by value)
  g.n = n;
  g.status = nullptr;
  int64_t total_tiles = 0;
  for (int i = 0; i < n; ++i) {
    const Prepared& t = items[i];
    WgradProblem& q = g.prob[i];
    if (g.status == nullptr) g.status = t.status;
    q.BT = static_cast<int>(t.bt);
    q.V = static_cast<int>(t.V);
    q.H = static_cast<int>(t.H);
    q.num_kb = static_cast<int>((t.bt + Cfg::kBK - 1) / Cfg::kBK);
    q.tiles_m = static_cast<int>((t.V + TILE_M * CG - 1) / (TILE_M * CG));
    q.tiles_n = static_cast<int>((t.H + TILE_N - 1) / TILE_N);
    q.ld_scale = static_cast<int>(t.ld_scale);
    q.dy = static_cast<const uint8_t*>(t.dy);
    q.x = static_cast<const uint8_t*>(t.x);
    q.ld_dy_bytes = t.ld_dy * 2;
    q.ld_x_bytes = t.ld_x * 2;
    q.m_scale = t.m_scale;
    q.v_scale = t.v_scale;
    q.m_absmax = t.m_absmax;
    q.v_absmax = t.v_absmax;
    q.hyper_dev = t.hyper_dev;
    q.hyper = t.hyper;
    total_tiles += static_cast<int64_t>(q.tiles_m) * q.tiles_n;
    int rc;
    // boxes of 128 rows x one swizzle row of a chunk; the same maps serve the loads and the stores
    if ((rc = encode_tmap_2d(&q.tm_w, t.W, Cfg::kWES, true, t.V, t.H, t.ld_w, WG::kBoxRowBytes / Cfg::kWES, 128,
                             WG::kSwizzle)) != FORGE_OK)
      return rc;
    q.tm_m = q.tm_w;
    q.tm_v = q.tm_w;
    if constexpr (Cfg::kNMom > 0) {
      using SG = BoxGeom<Cfg::kSRB>;
      if ((rc = encode_tmap_2d(&q.tm_m, t.m, Cfg::kSES, Cfg::kSES != 1, t.V, t.H, t.ld_state,
                               SG::kBoxRowBytes / Cfg::kSES, 128, SG::kSwizzle)) != FORGE_OK)
        return rc;
      if constexpr (Cfg::kNMom > 1) {
        if ((rc = encode_tmap_2d(&q.tm_v, t.v, Cfg::kSES, Cfg::kSES != 1, t.V, t.H, t.ld_state,
                                 SG::kBoxRowBytes / Cfg::kSES, 128, SG::kSwizzle)) != FORGE_OK)
          return rc;
      }
    }
    // operand panels: boxes of 64 columns x one pipeline stage of token rows, 128-byte swizzle; with no
    // tokens the operand maps are never used, valid ones are passed anyway
    q.tm_dy = q.tm_w;
    q.tm_x = q.tm_w;
    if (t.bt > 0) {
      if ((rc = encode_tmap_2d(&q.tm_dy, t.dy, 2, true, t.bt, t.V, t.ld_dy, 64, Cfg::kBK, 128)) != FORGE_OK) return rc;
      if ((rc = encode_tmap_2d(&q.tm_x, t.x, 2, true, t.bt, t.H, t.ld_x, 64, Cfg::kBK, 128)) != FORGE_OK) return rc;
    }
  }
  // One cluster per work unit; the hardware starts as many as fit (one CTA per SM) and the running
  // ones take over the units of the rest.  The units of the problems follow each other in the order
  // the problems were given.  A launch whose tiles would leave half of the SMs idle is cut into
  // 128-column halves throughout; otherwise the last `tail` tiles of the launch are, to shorten the
  // ragged end.
  const int64_t workers = sm_count / CG;
  int64_t halves = (2 * total_tiles <= workers) ? total_tiles : std::min<int64_t>(total_tiles, tail_halves(total_tiles, workers));
  int64_t units = 0;
  for (int i = n - 1; i >= 0; --i) {
    WgradProblem& q = g.prob[i];
    const int64_t tiles = static_cast<int64_t>(q.tiles_m) * q.tiles_n;
    const int64_t h = std::min<int64_t>(tiles, halves);
    halves -= h;
    q.split_from = static_cast<int>(tiles - h);
    q.num_units = static_cast<int>(tiles + h);
    units += tiles + h;
  }
  if (units * CG > 0x7fffffffLL) return fail(FORGE_ERR_SHAPE, "launch of %lld work units is too large", (long long)units);
  int base = 0;
  for (int i = 0; i < n; ++i) {
    g.prob[i].unit_base = base;
    base += g.prob[i].num_units;
  }
  g.num_units = base;
  const int grid = CG * g.num_units;
  auto kern = forge_wgrad_kernel<W_DT, ST, OPT, CG>;
  static std::atomic<bool> attr_set[64];   // per device: the shared-memory opt-in of this configuration has been made
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess)
      return fail(FORGE_ERR_CUDA, "cudaFuncSetAttribute(%d bytes): %s", Cfg::kSmemBytes, cudaGetErrorString(e));
    attr_set[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "wgrad kernel launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}

// CTA pairs are used whenever a weight of the launch has more than one 128-row tile;
// FORGE_CTA_PAIRS=0 in the environment keeps single CTAs (a tuning / bisecting aid, read once).
static bool pairs_enabled() {
  static const bool on = [] {
    const char* e = getenv("FORGE_CTA_PAIRS");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

template <int W_DT>
static int dispatch_wgrad(const Prepared* items, int n, int sm_count, cudaStream_t s) {
  const int opt = items[0].opt, st = items[0].st;
  bool pair = false;
  for (int i = 0; i < n; ++i) pair = pair || items[i].V > TILE_M;
  pair = pair && pairs_enabled() && sm_count >= 2;
#define FORGE_CASE(OPT_, ST_)                                                             \
  if (opt == OPT_ && st == ST_)                                                           \
    return pair ? launch_wgrad<W_DT, ST_, OPT_, 2>(items, n, sm_count, s)                 \
                : launch_wgrad<W_DT, ST_, OPT_, 1>(items, n, sm_count, s);
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

// Checks one argument block and fills `out`.  Launches nothing.  `*skip` is set for an empty
// parameter (V or H zero), which needs no work.
static int prepare(const ForgeWgradArgs& a, Prepared* out, bool* skip) {
  *skip = false;
  if (a.BT < 0 || a.V < 0 || a.H < 0) return fail(FORGE_ERR_INVALID_ARG, "negative dimension");
  if (a.V == 0 || a.H == 0) { *skip = true; return FORGE_OK; }  // empty parameter: nothing to update
  if (a.W == nullptr) return fail(FORGE_ERR_INVALID_ARG, "W is NULL");
  if (a.BT > 0 && (a.dY == nullptr || a.X == nullptr)) return fail(FORGE_ERR_INVALID_ARG, "dY or X is NULL");
  if (a.BT > (1 << 28) || a.V > (1ll << 30) || a.H > (1ll << 30)) return fail(FORGE_ERR_SHAPE, "dimension too large");
  if (a.w_dtype != FORGE_DT_BF16 && a.w_dtype != FORGE_DT_F32) return fail(FORGE_ERR_INVALID_ARG, "unknown W dtype %d", a.w_dtype);
  if (a.operand_dtype != FORGE_DT_BF16 && a.operand_dtype != FORGE_DT_F32)
    return fail(FORGE_ERR_INVALID_ARG, "unknown operand dtype %d", a.operand_dtype);
  const int opt = a.optimizer;
  int st = a.state.mode;
  if (opt < FORGE_OPT_ADAMW || opt > FORGE_OPT_LION) return fail(FORGE_ERR_INVALID_ARG, "unknown optimizer %d", opt);
  if (opt == FORGE_OPT_SGD) st = FORGE_ST_NONE;
  if (opt != FORGE_OPT_SGD && (st < FORGE_ST_F32 || st > FORGE_ST_FP8_TENSOR))
    return fail(FORGE_ERR_INVALID_ARG, "unknown state mode %d", st);
  if (a.hyper_device == nullptr && a.hyper.step < 1 && opt == FORGE_OPT_ADAMW)
    return fail(FORGE_ERR_INVALID_ARG, "step must be >= 1 (got %d)", a.hyper.step);
  if (a.hyper_device != nullptr && (reinterpret_cast<uintptr_t>(a.hyper_device) & 15u) != 0)
    return fail(FORGE_ERR_ALIGNMENT, "hyper_device is not 16-byte aligned");
  const int nm = num_moments(opt);
  if (nm > 0 && a.state.m == nullptr) return fail(FORGE_ERR_INVALID_ARG, "first moment buffer is NULL");
  if (nm > 1 && a.state.v == nullptr) return fail(FORGE_ERR_INVALID_ARG, "second moment buffer is NULL");
  const bool blockq = (st == FORGE_ST_INT8 || st == FORGE_ST_FP8_BLOCK);
  if (blockq) {
    if (a.state.qblock != 64) return fail(FORGE_ERR_SHAPE, "qblock must be 64 (got %d)", a.state.qblock);
    if (a.H % 64 != 0) return fail(FORGE_ERR_SHAPE, "H (%lld) must be divisible by qblock (64)", (long long)a.H);
    if (a.state.m_scale == nullptr || a.state.v_scale == nullptr) return fail(FORGE_ERR_INVALID_ARG, "scale arrays are NULL");
    if (a.state.ld_scale < a.H / 64) return fail(FORGE_ERR_INVALID_ARG, "ld_scale too small");
  }
  if (st == FORGE_ST_FP8_TENSOR) {
    if (a.state.m_scale == nullptr || a.state.v_scale == nullptr || a.state.m_absmax_next == nullptr ||
        a.state.v_absmax_next == nullptr)
      return fail(FORGE_ERR_INVALID_ARG, "fp8 per-tensor scale / absmax pointers are NULL");
  }
  if (a.BT > 0 && a.operand_dtype == FORGE_DT_F32) {
    const size_t need = forge_wgrad_scratch_bytes(a.BT, a.V, a.H, FORGE_DT_F32);
    if (a.scratch == nullptr || a.scratch_bytes < need)
      return fail(FORGE_ERR_SCRATCH, "fp32 operands need %zu bytes of scratch (got %zu)", need, a.scratch_bytes);
    if (!aligned16(a.scratch)) return fail(FORGE_ERR_ALIGNMENT, "scratch is not 16-byte aligned");
  }
  Prepared& t = *out;
  t.W = a.W; t.m = a.state.m; t.v = a.state.v;
  t.V = a.V; t.H = a.H; t.ld_w = a.ld_w; t.ld_state = a.state.ld_state;
  t.dy = a.dY; t.x = a.X; t.bt = a.BT; t.ld_dy = a.ld_dy; t.ld_x = a.ld_x;
  t.m_scale = a.state.m_scale;
  t.v_scale = a.state.v_scale;
  t.ld_scale = a.state.ld_scale;
  t.m_absmax = a.state.m_absmax_next;
  t.v_absmax = a.state.v_absmax_next;
  t.hyper = make_hyper(a.hyper);
  t.hyper_dev = static_cast<const Hyper*>(a.hyper_device);
  t.status = a.status;
  t.w_dtype = a.w_dtype; t.opt = opt; t.st = st;
  return FORGE_OK;
}

// fp32 operands: split into bf16 hi / lo parts in the caller's scratch (see split_f32_kernel) and
// point the problem at the stacked copies
static int split_operands(const ForgeWgradArgs& a, Prepared* t, cudaStream_t stream) {
  const int64_t bt_pad = (a.BT + 63) / 64 * 64;
  __nv_bfloat16* sa = static_cast<__nv_bfloat16*>(a.scratch);
  __nv_bfloat16* sb = sa + 3 * bt_pad * a.V;
  const int threads = 256;
  const int blocks_a = static_cast<int>(std::min<int64_t>((bt_pad * a.V + threads - 1) / threads, 148 * 8));
  const int blocks_b = static_cast<int>(std::min<int64_t>((bt_pad * a.H + threads - 1) / threads, 148 * 8));
  split_f32_kernel<<<blocks_a, threads, 0, stream>>>(static_cast<const float*>(a.dY), a.BT, a.V, a.ld_dy, bt_pad, sa, 0);
  split_f32_kernel<<<blocks_b, threads, 0, stream>>>(static_cast<const float*>(a.X), a.BT, a.H, a.ld_x, bt_pad, sb, 1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "operand split launch: %s", cudaGetErrorString(e));
  t->dy = sa; t->x = sb; t->bt = 3 * bt_pad; t->ld_dy = a.V; t->ld_x = a.H;
  return FORGE_OK;
}

}  // namespace forge

using namespace forge;

extern "C" size_t forge_wgrad_scratch_bytes(int64_t BT, int64_t V, int64_t H, int32_t operand_dtype) {
  if (operand_dtype != FORGE_DT_F32 || BT <= 0 || V <= 0 || H <= 0) return 0;
  const int64_t bt_pad = (BT + 63) / 64 * 64;
  return static_cast<size_t>(3 * bt_pad) * static_cast<size_t>(V + H) * sizeof(__nv_bfloat16);
}

extern "C" int forge_wgrad_update_group(const ForgeWgradArgs* args, int32_t count, void* cuda_stream) {
  if (count < 0) return fail(FORGE_ERR_INVALID_ARG, "forge_wgrad_update_group: negative count");
  if (count == 0) return FORGE_OK;
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_wgrad_update_group: args is NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // every block is checked before anything is launched: a bad entry leaves all weights untouched
  std::vector<Prepared> items;
  std::vector<int> source;
  items.reserve(count);
  source.reserve(count);
  for (int32_t i = 0; i < count; ++i) {
    Prepared t;
    bool skip = false;
    const int rc = prepare(args[i], &t, &skip);
    if (rc != FORGE_OK) return rc;
    if (skip) continue;
    items.push_back(t);
    source.push_back(i);
  }
  if (items.empty()) return FORGE_OK;
  const DeviceInfo* di = current_device_info();
  if (di == nullptr) return FORGE_ERR_CUDA;
  if (di->cc_major != 10) return fail(FORGE_ERR_DEVICE, "device has compute capability %d.%d; sm_100 is required", di->cc_major, di->cc_minor);
  for (size_t k = 0; k < items.size(); ++k) {
    const ForgeWgradArgs& a = args[source[k]];
    if (a.BT > 0 && a.operand_dtype == FORGE_DT_F32) {
      const int rc = split_operands(a, &items[k], stream);
      if (rc != FORGE_OK) return rc;
    }
  }
  // consecutive entries of one kernel configuration share a launch, MAX_GROUP at most
  size_t k = 0;
  while (k < items.size()) {
    size_t e = k + 1;
    while (e < items.size() && e - k < static_cast<size_t>(MAX_GROUP) && items[e].w_dtype == items[k].w_dtype &&
           items[e].opt == items[k].opt && items[e].st == items[k].st)
      ++e;
    const int n = static_cast<int>(e - k);
    const int rc = (items[k].w_dtype == FORGE_DT_BF16) ? dispatch_wgrad<DT_BF16>(&items[k], n, di->sm_count, stream)
                                                       : dispatch_wgrad<DT_F32>(&items[k], n, di->sm_count, stream);
    if (rc != FORGE_OK) return rc;
    k = e;
  }
  return FORGE_OK;
}

extern "C" int forge_wgrad_update(const ForgeWgradArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_wgrad_update: args is NULL");
  return forge_wgrad_update_group(args, 1, cuda_stream);
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant for fp32 operands.
//
// The fp32-operand path needs scratch for the bf16 hi/lo split of dY and X.  Some callers have no
// way to provide it: a plug-in invoked from inside a host framework's allocator callback (calling
// back into the allocator would re-enter it), or a job whose device memory was committed in full to
// a static plan at start-up.  For them the scratch is this fixed array inside the library image.
// Every GPU that loads the library carries it until the process exits.  All calls on a device share
// it and it keeps whatever the last call wrote; the split kernels overwrite every byte a call will
// read (padding rows included), so nothing needs clearing, but two calls that overlap on the GPU
// (different streams) race on it.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[FORGE_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device.  The symbol's name is only a host-side handle;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device (and once per
// calling thread, which also makes sure that thread has the device's context bound).
static int static_scratch_address(void** out) {
  static void* cached[64] = {};            // guarded by cache_mutex
  static std::mutex cache_mutex;
  static thread_local bool thread_ready[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return fail(FORGE_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(cache_mutex);
  if (cached[dev] == nullptr || !thread_ready[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(FORGE_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
    cached[dev] = ptr;
    thread_ready[dev] = true;
  }
  *out = cached[dev];
  return FORGE_OK;
}

extern "C" int forge_wgrad_update_static_scratch(const ForgeWgradArgs* args, void* cuda_stream) {
  if (args == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_wgrad_update_static_scratch: args is NULL");
  if (args->operand_dtype != FORGE_DT_F32)
    return fail(FORGE_ERR_INVALID_ARG, "forge_wgrad_update_static_scratch is for fp32 dY / X; bf16 operands need no "
                                       "scratch, call forge_wgrad_update");
  const size_t need = forge_wgrad_scratch_bytes(args->BT, args->V, args->H, FORGE_DT_F32);
  if (need > static_cast<size_t>(FORGE_STATIC_SCRATCH_BYTES))
    return fail(FORGE_ERR_SCRATCH,
                "problem needs %zu bytes of scratch but the built-in array holds %zu: 3 * roundup(BT, 64) * (V + H) * 2 "
                "must not exceed it; use forge_wgrad_update with caller scratch",
                need, static_cast<size_t>(FORGE_STATIC_SCRATCH_BYTES));
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != FORGE_OK) return rc;
  ForgeWgradArgs a = *args;
  a.scratch = scratch;
  a.scratch_bytes = static_cast<size_t>(FORGE_STATIC_SCRATCH_BYTES);
  return forge_wgrad_update(&a, cuda_stream);
}

static_assert(sizeof(forge::Hyper) <= FORGE_HYPER_DEVICE_BYTES, "packed hyper block too small");

extern "C" int forge_hyper_pack(const ForgeHyper* h, void* out) {
  if (h == nullptr || out == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_hyper_pack: null pointer");
  if (h->step < 1) return fail(FORGE_ERR_INVALID_ARG, "step must be >= 1 (got %d)", h->step);
  memset(out, 0, FORGE_HYPER_DEVICE_BYTES);
  const forge::Hyper packed = forge::make_hyper(*h);
  memcpy(out, &packed, sizeof(packed));
  return FORGE_OK;
}
