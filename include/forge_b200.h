/* forge_b200 -- C ABI of the B200 (sm_100a) fused weight-gradient + optimizer path.
 *
 * Plain C types only: device pointers, sizes, enums as int, hyper-parameters as float/double and a
 * CUDA stream passed as void*.  Every function returns FORGE_OK (0) or a negative FORGE_ERR_* code;
 * forge_last_error_string() gives the message of the last failure on the calling thread.  The
 * library allocates no device memory at run time; every buffer belongs to the caller.  (The library
 * image carries one fixed array of FORGE_STATIC_SCRATCH_BYTES per GPU, used only by
 * forge_wgrad_update_static_scratch.)  All launches go to the stream the caller passes and return
 * without synchronising.
 *
 * Shapes follow the reference: dY is (BT, V) "grad_output", X is (BT, H) "input", W and the
 * optimizer moments are (V, H); all row-major with the last dimension contiguous.
 */
#ifndef FORGE_B200_H_
#define FORGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FORGE_ABI_VERSION 3

/* error codes */
#define FORGE_OK 0
#define FORGE_ERR_INVALID_ARG (-1)  /* null pointer, unknown enum, negative size                  */
#define FORGE_ERR_ALIGNMENT (-2)    /* pointer not 16-byte aligned or row pitch not 16-byte sized */
#define FORGE_ERR_SHAPE (-3)        /* shape not supported (e.g. H % 64 != 0 with int8 moments)    */
#define FORGE_ERR_UNSUPPORTED (-4)  /* dtype / optimizer / state-mode combination not built        */
#define FORGE_ERR_CUDA (-5)         /* a CUDA runtime or driver call failed                        */
#define FORGE_ERR_DEVICE (-6)       /* device is not sm_100                                        */
#define FORGE_ERR_TIMEOUT (-7)      /* a kernel abandoned a bounded wait (see forge_read_status)   */
#define FORGE_ERR_SCRATCH (-8)      /* scratch buffer missing or too small                         */

/* element types of dY/X and of W */
#define FORGE_DT_BF16 0
#define FORGE_DT_F32 1

/* optimizers */
#define FORGE_OPT_ADAMW 0
#define FORGE_OPT_SGD 1   /* plain SGD with decoupled decay, no state                       */
#define FORGE_OPT_SGDM 2  /* SGD with momentum (one moment buffer), optional Nesterov       */
#define FORGE_OPT_LION 3  /* Lion (one moment buffer)                                       */

/* storage of the optimizer moments */
#define FORGE_ST_NONE 0
#define FORGE_ST_F32 1
#define FORGE_ST_BF16 2
#define FORGE_ST_INT8 3       /* int8 codes + fp32 absmax scale per (row, 64 columns)            */
#define FORGE_ST_FP8_BLOCK 4  /* e4m3 codes (m and v) + fp32 absmax scale per (row, 64 columns)  */
#define FORGE_ST_FP8_TENSOR 5 /* e4m3 m, e5m2 v, one fp32 scale per tensor, delayed scaling      */

/* flags */
#define FORGE_FLAG_NONE 0u

/* Hyper-parameters of one update.  `step` is the 1-based count of updates of this parameter; the
 * bias corrections 1 - beta^step are evaluated in double and narrowed to float, as the reference
 * does (src/fused_grad_optimizer/kernel.py:1367-1368). */
typedef struct ForgeHyper {
  double lr;
  double beta1;
  double beta2;
  double eps;
  double weight_decay;
  double momentum; /* FORGE_OPT_SGDM only */
  int32_t nesterov;
  int32_t step;
} ForgeHyper;

/* The optimizer state of one (V, H) parameter.  Unused pointers are NULL. */
typedef struct ForgeState {
  int32_t mode;      /* FORGE_ST_*                                                             */
  int32_t qblock;    /* columns per quantisation block; must be 64 for INT8 / FP8_BLOCK         */
  void* m;           /* first moment / momentum buffer, (V, H), element type by `mode`          */
  void* v;           /* second moment, (V, H)                                                   */
  int64_t ld_state;  /* row pitch of m and v in elements                                        */
  float* m_scale;    /* INT8 / FP8_BLOCK: (V, H/qblock) fp32; FP8_TENSOR: one fp32 scalar       */
  float* v_scale;
  int64_t ld_scale;  /* row pitch of the scale arrays in floats (INT8 / FP8_BLOCK)              */
  float* m_absmax_next; /* FP8_TENSOR: running max |m'| of this step (atomic max), one scalar   */
  float* v_absmax_next;
} ForgeState;

/* Arguments of the fused weight-gradient + optimizer update. */
typedef struct ForgeWgradArgs {
  const void* dY;    /* (BT, V) row-major                                                       */
  const void* X;     /* (BT, H) row-major                                                       */
  void* W;           /* (V, H) row-major, updated in place                                      */
  int64_t BT, V, H;
  int64_t ld_dy, ld_x, ld_w; /* row pitches in elements                                         */
  int32_t operand_dtype;     /* FORGE_DT_* of dY and X                                          */
  int32_t w_dtype;           /* FORGE_DT_* of W                                                 */
  int32_t optimizer;         /* FORGE_OPT_*                                                     */
  uint32_t flags;
  ForgeState state;
  ForgeHyper hyper;
  void* scratch;             /* only for fp32 operands: see forge_wgrad_scratch_bytes           */
  size_t scratch_bytes;
  int32_t* status;           /* optional device word; a kernel that abandons a wait writes its
                                code here (0 = ok); see forge_read_status                       */
  const void* hyper_device;  /* optional: FORGE_HYPER_DEVICE_BYTES of DEVICE memory holding the output
                                of forge_hyper_pack.  When non-NULL the kernel reads its
                                hyper-parameters from there at run time and `hyper` is ignored, so
                                a captured CUDA graph can be replayed with a new lr / step by
                                rewriting that block before each replay.                         */
} ForgeWgradArgs;

/* Bytes of the packed hyper-parameter block. */
#define FORGE_HYPER_DEVICE_BYTES 64

/* Narrows `h` exactly as forge_wgrad_update does internally (bias corrections in double, then
 * float) and writes the FORGE_HYPER_DEVICE_BYTES block the kernels read into HOST memory `out`;
 * copy it to the device buffer passed as ForgeWgradArgs.hyper_device.  No reference counterpart
 * (the reference passes hyper-parameters as kernel arguments, src/fused_grad_optimizer/
 * kernel.py:1367-1368, which pins them into a captured graph). */
int forge_hyper_pack(const ForgeHyper* h, void* out);

/* Fused dW = dY^T X and in-place optimizer update of W and its moments; no gradient tensor is
 * written to memory.  Replaces the reference's fused_grad_adamw / fused_grad_sgd /
 * fused_grad_adamw_int8state / fused_grad_adamw_fp8state
 * (src/fused_grad_optimizer/kernel.py:1342-1455, :1319-1339, :1487-1539;
 * src/fused_grad_optimizer/kernel_fp8_state.py:343-392).  Must be enqueued after the dX GEMM that
 * reads the same W on the same stream (src/fused_grad_optimizer/autograd.py:50-55). */
int forge_wgrad_update(const ForgeWgradArgs* args, void* cuda_stream);

/* Weights one kernel launch of forge_wgrad_update_group covers. */
#define FORGE_MAX_GROUP 16

/* The fused update of `count` weights in as few launches as possible: consecutive entries that agree
 * in w_dtype, optimizer and state mode share one launch, FORGE_MAX_GROUP at most, so that the fixed
 * start-up and ragged end of a launch are paid once per group instead of once per weight (the q / k /
 * v projections of a layer, gate / up, or all seven projections of a decoder layer).  Entries may
 * differ in BT, V, H, hyper-parameters and operands.  The reference launches one kernel per linear
 * from _apply_fused (src/fused_grad_optimizer/autograd.py:94-144); this replaces a run of those
 * calls.  Every entry is checked before anything is launched: on an error no weight has been
 * touched.  The result of each weight is bit-identical to forge_wgrad_update on that entry alone.
 * Entries must not alias each other's W or state.  The work units follow the order of the entries;
 * put the largest weights first.  A kernel that abandons a wait reports through the first non-NULL
 * `status` of its launch. */
int forge_wgrad_update_group(const ForgeWgradArgs* args, int32_t count, void* cuda_stream);

/* Bytes of scratch forge_wgrad_update needs for the given operand type (0 for bf16 operands; fp32
 * operands are split into bf16 high/low parts in scratch before the GEMM). */
size_t forge_wgrad_scratch_bytes(int64_t BT, int64_t V, int64_t H, int32_t operand_dtype);

/* Size of the scratch array built into the library for forge_wgrad_update_static_scratch. */
#define FORGE_STATIC_SCRATCH_BYTES (32u << 20)

/* forge_wgrad_update for fp32 dY / X without any caller-provided scratch and without a single
 * allocation: the bf16 hi/lo split goes to a fixed FORGE_STATIC_SCRATCH_BYTES array inside the
 * library (args->scratch and args->scratch_bytes are ignored).  This entry point has no counterpart
 * in the reference.  It exists for callers that cannot allocate device memory where they call it
 * from: a plug-in running inside a host framework's allocator callback, or a job whose memory was
 * handed out in full to a static plan at start-up.
 *   - Limit: forge_wgrad_scratch_bytes(BT, V, H, FORGE_DT_F32) = 3 * roundup(BT, 64) * (V + H) * 2
 *     must not exceed FORGE_STATIC_SCRATCH_BYTES (e.g. BT = 512 with V + H <= 10922); larger problems
 *     return FORGE_ERR_SCRATCH.  bf16 operands return FORGE_ERR_INVALID_ARG (they need no scratch).
 *   - The first call on each device (and from each new thread) looks up the array's device address;
 *     make that first call before starting a stream capture.
 *   - Each GPU that loads the library holds the array until the process ends.  All calls on a device
 *     share it and it keeps the previous call's contents; every byte a call reads is written by that
 *     call first, but calls that overlap on the GPU (two streams) race on it -- serialise them.
 * Results are identical to forge_wgrad_update given the same arguments. */
int forge_wgrad_update_static_scratch(const ForgeWgradArgs* args, void* cuda_stream);

/* Arguments of the optimizer-only update on a materialised gradient. */
typedef struct ForgeOptimArgs {
  const void* grad;  /* (V, H) row-major gradient                                                */
  void* W;           /* (V, H) row-major, updated in place                                       */
  int64_t V, H;
  int64_t ld_grad, ld_w;
  int32_t grad_dtype; /* FORGE_DT_*                                                              */
  int32_t w_dtype;
  int32_t optimizer;
  uint32_t flags;
  ForgeState state;
  ForgeHyper hyper;
} ForgeOptimArgs;

/* Optimizer update from a gradient that already exists in memory (gradient accumulation, layers
 * that opt out of the fused backward).  Replaces optimizer_only_adamw /
 * optimizer_only_adamw_int8state (src/fused_grad_optimizer/kernel.py:1458-1484, :1542-1575) and the
 * SGD branch of _apply_precomputed (src/fused_grad_optimizer/autograd.py:153-156).  Shares the
 * per-element arithmetic of forge_wgrad_update bit for bit. */
int forge_optimizer_update(const ForgeOptimArgs* args, void* cuda_stream);

/* Delayed-scaling bookkeeping of FORGE_ST_FP8_TENSOR before an update, on the device and without a
 * host synchronisation: scale <- clamp(absmax_next, 1e-8) / MAX, capped at twice the previous scale
 * when that is positive; absmax_next <- 0.  Replaces FusedOptimizerState.pre_step_fp8
 * (src/fused_grad_optimizer/state.py:132-157), which reads both scales back to the host. */
int forge_fp8_prestep(float* m_scale, float* v_scale, float* m_absmax_next, float* v_absmax_next,
                      void* cuda_stream);

/* dX = dY W : (BT, V) x (V, H) -> (BT, H), bf16 in, fp32 accumulate, bf16 out.  Replaces
 * `grad_input = grad_output @ weight` (src/fused_grad_optimizer/autograd.py:55). */
int forge_dgrad(const void* dY, const void* W, void* dX, int64_t BT, int64_t V, int64_t H,
                int64_t ld_dy, int64_t ld_w, int64_t ld_dx, int32_t* status, void* cuda_stream);

/* One (dY_i, W_i) pair of a summed input gradient. */
typedef struct ForgeDgradSegment {
  const void* dY;    /* (BT, V) bf16 */
  const void* W;     /* (V, H) bf16 */
  int64_t V;
  int64_t ld_dy, ld_w;
} ForgeDgradSegment;

/* dX = sum_i dY_i W_i over up to 4 pairs in one launch, the accumulator staying in tensor memory: the
 * input gradient of linears that share their input (q / k / v; gate / up).  Replaces the sum autograd
 * forms from one `grad_output @ weight` per linear (src/fused_grad_optimizer/autograd.py:55). */
int forge_dgrad_sum(const ForgeDgradSegment* segments, int32_t count, void* dX, int64_t BT, int64_t H, int64_t ld_dx,
                    int32_t* status, void* cuda_stream);

/* The row-sharded tensor-parallel mode's partial input gradient with its reduce-scatter fused into the
 * GEMM (no counterpart in the reference, which has no distributed code).  The columns of dX are cut
 * into `world` feature blocks of H / world columns (a multiple of 128); every 128 x 128 output tile is
 * stored from the epilogue straight into the receive buffer of the rank that owns its block -- slot
 * [rank] of that rank's (world, BT, H / world) bf16 buffer -- with plain peer stores; when the launch's
 * last tile is out, this rank's arrival word on every owner is set to *epoch.
 *   slots[o], arrivals[o]: rank o's receive buffer and its `world` arrival words, mapped into this
 *     process (CUDA IPC or any peer mapping); entries [rank] are this rank's own memory.
 *   counter: a local device word, zero before the first launch that uses it; the kernel leaves it zero.
 *   epoch: a local device word holding the value to raise; change it between steps (e.g. add one inside
 *     the captured graph) so that forge_reduce_slots can tell this step's arrival from the last one's.
 * A receive buffer may be reused only after every rank has finished reading it (a collective of the
 * next forward pass, or a barrier, between two uses is enough). */
typedef struct ForgeDgradScatterArgs {
  const ForgeDgradSegment* segments;
  int32_t count;
  int64_t BT, H;
  void* const* slots;
  uint32_t* const* arrivals;
  uint32_t* counter;
  const uint32_t* epoch;
  int32_t rank, world;
  int32_t* status;
  int32_t all_ranks;   /* 1: a fused ALL-REDUCE instead -- every tile is stored into slot [rank] of EVERY rank's
                          buffer, which is then (world, BT, H) wide, and forge_reduce_slots is called with
                          block_cols = H; for a linear set whose input is replicated (q / k / v, gate / up) */
} ForgeDgradScatterArgs;
int forge_dgrad_scatter(const ForgeDgradScatterArgs* args, void* cuda_stream);

/* The owner's half of the fused reduce-scatter: waits (bounded; on expiry code 211 goes to *status)
 * until all `world` arrival words equal *epoch, then out[m, c] = sum over src of slots[src][m, c], added
 * in rank order in fp32 (bit-reproducible), as bf16. */
int forge_reduce_slots(const void* slots, const uint32_t* arrivals, const uint32_t* epoch, void* out, int64_t BT,
                       int64_t block_cols, int64_t ld_out, int32_t world, int32_t* status, void* cuda_stream);

/* How long forge_reduce_slots waits for its arrival words before it gives up (default: two seconds;
 * process-wide; tests shorten it). */
int forge_set_arrival_wait_ns(uint64_t ns);

/* The forward product of the row-sharded mode with its all-gathers fused in (no counterpart in the
 * reference: Y = X W^T is `F.linear`, src/fused_grad_optimizer/autograd.py:34, and it has no distributed
 * code).  Three calls:
 *
 * forge_push_block: copies this rank's (BT, cols) bf16 block into EVERY rank's gathered (BT, ld_dst)
 *   matrix at column `col` with plain peer stores, then sets arrival word [rank] on every rank to
 *   *epoch.  dst[o], arrivals[o]: rank o's matrix and its `world` arrival words mapped into this
 *   process; counter: a local zero word (left zero).  This is the all-gather of a feature-sharded X.
 *
 * forge_linear_gathered: Y = X W_r^T, X the gathered (BT, H) matrix in LOCAL memory that the ranks fill
 *   with forge_push_block, cut into `world` equal feature blocks; W_r this rank's (V_r, H) rows.  The
 *   GEMM starts with the own block and waits for each other block's arrival word (x_arrivals[src] ==
 *   *epoch; bounded like every wait, code 211) only when it gets there.  x_arrivals == NULL: X is
 *   complete already.  Output: y != NULL -> local (BT, V_r) bf16 with row pitch ld_y.  y == NULL -> every
 *   tile is stored into EVERY rank's gathered (BT, y_pitch) output at column y_col (the all-gather of the
 *   row-sharded output: y_dst[o], y_arrivals[o], y_counter as in forge_push_block), to be picked up with
 *   forge_collect.  H / world must be a multiple of 8, y_col and y_pitch too.
 *
 * forge_collect: waits (bounded, code 211) until all `world` arrival words equal *epoch, then copies
 *   the gathered (BT, cols) matrix to `out`. */
int forge_push_block(const void* src, int64_t BT, int64_t cols, int64_t ld_src, void* const* dst, int64_t col,
                     int64_t ld_dst, uint32_t* const* arrivals, uint32_t* counter, const uint32_t* epoch,
                     int32_t rank, int32_t world, int32_t* status, void* cuda_stream);

typedef struct ForgeLinearGatheredArgs {
  const void* X;                 /* local gathered input (BT, H), row pitch ld_x */
  const void* W;                 /* this rank's rows (V_r, H), row pitch ld_w */
  int64_t BT, H, V_r, ld_x, ld_w;
  const uint32_t* x_arrivals;    /* local: `world` words, or NULL */
  const uint32_t* epoch;
  int32_t rank, world;
  void* y;                       /* local output, or NULL for the pushed form */
  int64_t ld_y;
  void* const* y_dst;            /* pushed form: every rank's gathered output, column offset and row pitch */
  int64_t y_col, y_pitch;
  uint32_t* const* y_arrivals;
  uint32_t* y_counter;
  int32_t* status;
} ForgeLinearGatheredArgs;
int forge_linear_gathered(const ForgeLinearGatheredArgs* args, void* cuda_stream);

int forge_collect(const void* gathered, int64_t ld_gathered, const uint32_t* arrivals, const uint32_t* epoch, void* out,
                  int64_t BT, int64_t cols, int64_t ld_out, int32_t world, int32_t* status, void* cuda_stream);

/* RMSNorm recomputation for linears that fold their preceding norm (the normalised activation is not
 * kept between forward and backward): y = bf16(gamma * (x * rsqrt(mean(x^2) + eps))), fp32 inside;
 * x, gamma, y bf16; x and y (rows, H) row-major, H a multiple of 8 and at most 16384.  Replaces
 * _rmsnorm_forward (src/fused_grad_optimizer/fused_rmsnorm_linear.py:32-41). */
int forge_rmsnorm_forward(const void* x, const void* gamma, void* y, int64_t rows, int64_t H, int64_t ld_x,
                          int64_t ld_y, double eps, void* cuda_stream);

/* Backward of the same norm: grad_x = g gamma rrms - x (sum_h g gamma x) rrms^3 / H (bf16) and
 * grad_gamma = sum_rows g x rrms, written (accumulate = 0) or added (accumulate = 1) to grad_gamma of
 * type grad_gamma_dtype (FORGE_DT_BF16 or FORGE_DT_F32).  The column sums are reduced in two
 * fixed-order stages through `scratch` (forge_rmsnorm_backward_scratch_bytes), so results are
 * bit-reproducible.  Replaces _rmsnorm_backward (fused_rmsnorm_linear.py:44-62). */
int forge_rmsnorm_backward(const void* x, const void* gamma, const void* grad_y, void* grad_x, void* grad_gamma,
                           int32_t grad_gamma_dtype, int32_t accumulate, int64_t rows, int64_t H, int64_t ld_x,
                           int64_t ld_gy, int64_t ld_gx, double eps, void* scratch, size_t scratch_bytes,
                           void* cuda_stream);
size_t forge_rmsnorm_backward_scratch_bytes(int64_t rows, int64_t H);

/* Bytes of optimizer state the allocator must provide for a (V, H) parameter: the moment arrays
 * and, separately, the scale arrays (src/fused_grad_optimizer/state.py:95-130). */
int forge_state_bytes(int32_t optimizer, int32_t mode, int64_t V, int64_t H, int32_t qblock,
                      size_t* moment_bytes_each, size_t* scale_bytes_each, int32_t* num_moments);

/* Copies the device status word to the host after synchronising the stream and clears it.
 * Returns FORGE_OK, or FORGE_ERR_TIMEOUT with the kernel's code in *code_out. */
int forge_read_status(int32_t* status, int32_t* code_out, void* cuda_stream);

/* Self-test of the failure path, for test suites: launches one small kernel whose bounded wait (the
 * same routine the update kernels wait with) is on a barrier nothing ever signals.  After `limit_ns`
 * (1 ns .. 1 s) the wait gives up, the kernel writes code 190 to *status and ends normally; a following
 * forge_read_status returns FORGE_ERR_TIMEOUT with that code and clears the word.  Nothing faults and
 * the context stays usable.  No reference counterpart (the reference has no device-side waits). */
int forge_selftest_wait_timeout(int32_t* status, uint64_t limit_ns, void* cuda_stream);

/* Message of the last error on the calling thread (never NULL). */
const char* forge_last_error_string(void);

/* FORGE_ABI_VERSION the library was built with. */
int forge_abi_version(void);

#ifdef __cplusplus
}
#endif

#endif /* FORGE_B200_H_ */
