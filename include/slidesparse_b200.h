/*
 * slidesparse_b200.h -- C ABI of the B200 (sm_100a) sparse W8A8 projection library.
 *
 * Every entry point takes plain pointers and sizes (no torch types), an explicit CUDA stream
 * (a cudaStream_t passed as void*; NULL = legacy default stream) and returns 0 on success or a
 * negative SS_E_* code; ss_last_error() gives the message of the calling thread's last failure.
 * Device pointers must belong to the device that is current when the call is made.  Nothing here
 * synchronises the stream or allocates device memory unless the comment of the entry says so.
 *
 * The comment above each declaration names the reference interface it replaces, as
 * file:line inside the SlideSparse-Diffusion source tree.
 *
 * Formats shared by all entries (mode group l in {4,6,8} for 2:4 / 4:6 / 6:8):
 *   valid = ceil(k/l) * (l/2-1) * 4      lifted K'        (packing.py:15-20)
 *   pk    = ceil128(valid)                padded K'
 *   pm    = ceil32(m), pn = ceil32(n)
 *   q        int8  [pm, pk]   quantised, slide-expanded activations, rows m..pm-1 zero
 *   sa       fp32  [pm]       per-token scales, rows m..pm-1 are 1.0
 *   packed   int8  [pn, pk/2] 2:4-compressed weights, bit-identical to the reference's
 *   metadata int32 [pn*pk/32] 4-bit index pairs, one nibble per quartet.  "raw" order is the
 *            reference's pre-reorder array (row-major [pn, pk/32], quartet g of a row in word g/8
 *            at bit 4*(g%8)).  The "b200" order, which the GEMM consumes, stores each block of
 *            32 rows x 128 lifted columns as 512 contiguous bytes:
 *              word(row r, raw column c) -> ((r/32)*(pk/128) + c/4)*128 + (r%32)*4 + c%4
 */
#ifndef SLIDESPARSE_B200_H
#define SLIDESPARSE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SS_OK 0
#define SS_E_ARG (-1)      /* contract violation: shape, alignment, null pointer, mode        */
#define SS_E_CUDA (-2)     /* a CUDA runtime/driver call failed (message has the CUDA string) */
#define SS_E_FORMAT (-3)   /* weight violates the (l-2):l or 2:4 structure                    */
#define SS_E_HANDLE (-4)   /* unknown or released plan handle                                 */
#define SS_E_DEVICE (-5)   /* a kernel reported a bounded wait that ran out                   */
#define SS_E_LIMIT (-6)    /* size beyond a stated maximum of the entry point                 */

/* Message for the calling thread's most recent non-zero return.  Never NULL. */
const char* ss_last_error(void);

/* Library/hardware facts.  out[0..7] = {abi version, compiled arch (100), device cc major,
 * cc minor, SM count, max opt-in shared memory per block, TMEM columns per SM (512),
 * GEMM kernel threads}.  Replaces the device gate and resource report of
 * csrc/dualscale_sm80.cu:282-318 (configure).  device < 0 skips the device fields (CPU-only use). */
int ss_query(int device, int64_t* out, int n_out);

/* (valid, pk) for logical width k.  packing.py:15-20 (lifted_k, alignment 128). */
int ss_lifted_k(int64_t k, int group, int64_t* valid, int64_t* pk);

/* ---- offline packer, host side --------------------------------------------------------- */

/* Exact (l-2):l -> overlapping 2:4 window expansion of an int8 weight [n,k] into [n,valid].
 * packing.py:23-52 (slide_weight): increasing window, then increasing lane; SS_E_FORMAT if a
 * group holds more than l-2 nonzeros. */
int ss_slide_weight_cpu(const int8_t* qweight, int64_t n, int64_t k, int group, int8_t* lifted);

/* 2:4 compression of a lifted weight [n,kl] (kl <= pk, pk % 128 == 0) into packed [pn,pk/2] and
 * metadata.  meta_raw and meta_b200 may each be NULL.  csrc/dualscale_sm80.cu:254-274 (pack_cpu,
 * values + raw words); the SM80 reorder of :275-278 is replaced by the b200 order above. */
int ss_pack_cpu(const int8_t* lifted, int64_t n, int64_t kl, int64_t pk,
                int8_t* packed, int32_t* meta_raw, int32_t* meta_b200);

/* Convert metadata between the raw and the b200 order (to_b200 != 0: raw -> b200). */
int ss_meta_convert(const int32_t* src, int32_t* dst, int64_t pn, int64_t pk, int to_b200);

/* ---- offline packer, device side -------------------------------------------------------- */

/* Per-output-channel symmetric INT8 grid of an already pruned weight: scale = 2*rowabsmax/255
 * (1 if the row is all zero), q = clamp(rint(w/scale), -128, 127).  w is fp32 [n,k] on the
 * device.  diffusion_research/reconstruction.py:41-53 (channel_scales, round_signed). */
int ss_weight_grid_device(const float* w, int64_t n, int64_t k, int8_t* qweight, float* scales,
                          void* stream);

/* slide_weight + pack_cpu in one kernel on the device: qweight int8 [n,k] -> packed [pn,pk/2],
 * metadata (b200 order).  status (device int32[1], zeroed by the caller) is set to 1 if any
 * group violates the (l-2):l structure.  packing.py:23-52 + csrc/dualscale_sm80.cu:254-274. */
int ss_pack_device(const int8_t* qweight, int64_t n, int64_t k, int group,
                   int8_t* packed, int32_t* meta_b200, int32_t* status, void* stream);

/* ---- weight preparation: fixed-order shared-curvature pruning with joint INT8 rounding ------ */

/* One column block [start, start+width) of compress (diffusion_research/reconstruction.py:86-112):
 * w fp32 [rows,columns] on the device, updated in place to the finalised values of the block;
 * upper fp32 [columns,columns] is the shared factor (factor_hessian, :18-39); scales [rows];
 * zeros uint8 [rows,columns] receives the selected zeros of the block, errors [rows,width] the
 * per-column errors, losses [rows] accumulates the proxy loss.  joint != 0 rounds each column to
 * the INT8 grid as it is finalised ("joint"), 0 leaves it ("prune_then_rtn").  start must be a
 * multiple of group and width at most ss_obs_max_blocksize(). */
int ss_obs_block(float* w, int64_t rows, int64_t columns, int64_t start, int64_t width,
                 const float* upper, const float* scales, int group, int joint,
                 uint8_t* zeros, float* errors, float* losses, void* stream);

/* w[:, start+width:] -= errors @ upper[start:start+width, start+width:], each sum taken as
 * fma(e, u, acc) in increasing k.  diffusion_research/reconstruction.py:113-114. */
int ss_obs_trailing(float* w, int64_t rows, int64_t columns, int64_t start, int64_t width,
                    const float* upper, const float* errors, void* stream);

/* Export of compress (diffusion_research/reconstruction.py:117-127): qweight = clamp(rint(w/scale))
 * with the selected zeros forced to 0.  status (device int32[1], zeroed by the caller) gets bit 0
 * if check_grid and some qweight*scale differs from w, bit 1 if a complete group of `group`
 * columns holds more than group-2 nonzeros. */
int ss_obs_finish(const float* w, const float* scales, const uint8_t* zeros, int64_t rows,
                  int64_t columns, int group, int check_grid, int8_t* qweight, int32_t* status,
                  void* stream);

/* Widest column block ss_obs_block accepts (shared-memory bound).  No counterpart in the reference. */
int ss_obs_max_blocksize(void);

/* ---- front-end: dynamic per-token quantisation + slide expansion ------------------------ */

/* x: BF16 [m,k], unit column stride, row stride x_row_stride elements.  Writes q [pm,pk] and
 * sa [pm] in one pass.  csrc/projection_sm80.cu:8-88,99-120 (quant_lift, quantize);
 * runtime.py:72-95 (quantize_lift). */
int ss_quantize_lift(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                     int8_t* q, float* sa, void* stream);

/* ---- GEMM: 2:4 sparse INT8 tcgen05 contraction with fused dequant epilogue --------------- */

/* out[m,n] (BF16, row stride out_row_stride elements) =
 *   bf16( fma(float(acc), sa[tok]*sw[ch], bias[ch]) [+ float(addend[tok,ch])] ),
 * acc = exact int32 dot of q[tok,:] with the decompressed weight row ch.  bias and addend may be
 * NULL.  metadata is in b200 order.  csrc/dualscale_sm80.cu:320-398 (launch, run) and :72-187
 * (scaled, DirectEpilogue). */
int ss_gemm_run(const int8_t* q, const int8_t* packed, const int32_t* meta_b200,
                const float* sa, const float* sw, const float* bias,
                const void* addend_bf16, int64_t addend_row_stride,
                void* out_bf16, int64_t out_row_stride,
                int64_t m, int64_t n, int64_t pm, int64_t pn, int64_t pk, void* stream);

/* Same contraction, raw int32 accumulators to acc[m,n] (row stride n).
 * integrations/cachequant/csrc/native_sparse_int32_sm80.cu:38-62,112-133. */
int ss_gemm_int32(const int8_t* q, const int8_t* packed, const int32_t* meta_b200,
                  int32_t* acc, int64_t m, int64_t n, int64_t pm, int64_t pn, int64_t pk,
                  void* stream);

/* Front-end + GEMM in one call.  q_scratch [pm,pk] and sa_scratch [pm] are caller-provided
 * device scratch.  csrc/projection_sm80.cu:142-148 (projection). */
int ss_projection(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                  const int8_t* packed, const int32_t* meta_b200,
                  const float* sw, const float* bias,
                  const void* addend_bf16, int64_t addend_row_stride,
                  int64_t n, int64_t pn,
                  int8_t* q_scratch, float* sa_scratch,
                  void* out_bf16, int64_t out_row_stride, void* stream);

/* Front-end with a fused element-wise prologue, and the projection built on it.
 * No counterpart in the reference, which runs these neighbours of the projection as separate PyTorch kernels
 * (adaLN-modulated LayerNorm before QKV / FFN-in, GELU before FFN-out): the row is rewritten in
 * registers before it is quantised, so the neighbour costs no extra pass over HBM.
 *   prologue 0  none (identical to ss_quantize_lift / ss_projection)
 *   prologue 1  y = ((x - mean) * rstd) * (1 + scale[b]) + shift[b], mean / biased variance over
 *               the k elements of the row, rstd = 1 / sqrt(var + eps), b = row / rows_per_batch;
 *               shift, scale: BF16 [ceil(m / rows_per_batch), k], rows mod_row_stride elements
 *               apart (>= k, multiple of 8), 16-byte aligned
 *   prologue 2  y = gelu_tanh(x) = 0.5 x (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3)))
 * y is rounded to BF16 and then quantised exactly as ss_quantize_lift quantises a BF16 input.
 * Needs 16-byte aligned rows and k % 8 == 0.  Prologue 1 uses separately rounded fp32 operations
 * in a fixed order, which the numpy oracle restates bit for bit; prologue 2 uses the hardware tanh
 * approximation (relative error 2^-11) and is exact to floating-point tolerance only:
 * |y - gelu_tanh(x)| <= 2.5e-4 |x| before the BF16 rounding. */
int ss_quantize_lift_fused(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                           int prologue, const void* shift_bf16, const void* scale_bf16,
                           int64_t mod_row_stride, int64_t rows_per_batch, float eps,
                           int8_t* q, float* sa, void* stream);
/* ss_quantize_lift_fused followed by the GEMM.  No counterpart in the reference (see above);
 * the remaining arguments are those of ss_projection, plus an optional gated accumulation, the
 * other element-wise neighbour of an FFN-out projection: with gate_bf16 != NULL (BF16
 * [ceil(m / rows_per_batch), n], rows gate_row_stride elements apart) the kernel does not store y
 * but adds bf16(gate[row / rows_per_batch, c] * y32[row, c]) to out_bf16 in place (y32 = the fp32
 * value fma(acc, sa*sw, bias) before its BF16 rounding; the addition is a BF16 round-to-nearest
 * add done by a TMA reduction), i.e. out is the residual stream.  Needs rows_per_batch % 32 == 0,
 * a 16-byte aligned out and row pitch, and no addend. */
int ss_projection_fused(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                        int prologue, const void* shift_bf16, const void* scale_bf16,
                        int64_t mod_row_stride, int64_t rows_per_batch, float eps,
                        const int8_t* packed, const int32_t* meta_b200,
                        const float* sw, const float* bias,
                        const void* addend_bf16, int64_t addend_row_stride,
                        const void* gate_bf16, int64_t gate_row_stride,
                        int64_t n, int64_t pn,
                        int8_t* q_scratch, float* sa_scratch,
                        void* out_bf16, int64_t out_row_stride, void* stream);

/* Tensor-parallel form of ss_projection.  No counterpart in the reference (which is single-GPU).
 * This rank computes its column shard y[m, n] (n = the shard's channels) and the GEMM epilogue
 * stores every tile to `count` destinations instead of one: destinations[g] is the address, in
 * this process's address space, of element [0, first column of this shard] of rank g's copy of
 * the gathered [m, N] output (this rank's own copy included; peer copies mapped through CUDA IPC
 * or symmetric memory), all with the row pitch out_row_stride (elements, a multiple of 8) and
 * 16-byte aligned.  The all-gather of the N-split variant thus happens inside the kernel, tile by
 * tile, as plain TMA stores over NVLink (no multicast); the caller orders the launch between two
 * cross-GPU barriers (nobody still reads the buffers before; every shard has landed after). */
int ss_projection_peers(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                        const int8_t* packed, const int32_t* meta_b200,
                        const float* sw, const float* bias,
                        int64_t n, int64_t pn,
                        int8_t* q_scratch, float* sa_scratch,
                        const void* const* destinations, int count, int64_t out_row_stride,
                        void* stream);

/* Diagnostic.  No counterpart in the reference.  Runs the GEMM kernel itself (clusters of two CTAs,
 * TMA producer, metadata copies, the real tile walk) on scratch operands of the given problem size
 * and returns the cycles per pipeline stage (256 lifted columns = four tcgen05.mma.sp of the pair)
 * that cluster 0 needed for its whole tile loop, with parts of the kernel switched off:
 *   flags bit 0  no MMAs are issued (commits only): the shared-memory feed from L2 alone
 *   flags bit 1  the epilogue hands every accumulator straight back: the main loop alone
 *   flags bit 2  the epilogue runs but does not issue its TMA stores (the output stays unwritten)
 *   flags bit 3  the epilogue only loads the accumulator from TMEM (no math, staging or stores)
 * token_tile 0 lets the library choose (including the weights-resident form); 128 / 192 / 224 /
 * 240 / 256 force a tile.  Allocates and frees its operands with cudaMalloc and synchronises the
 * device.  This is how the ceiling of the main loop's dataflow is measured, as opposed to argued. */
int ss_micro_pair_rate(int64_t m, int64_t n, int64_t pk, int token_tile, int flags,
                       double* cycles_per_stage, int64_t* stages);

/* Diagnostic.  No counterpart in the reference.  Proves the exit path of the bounded waits without
 * starving a real kernel: one warp waits, for at most limit_ns (1 ns .. 100 ms), on an mbarrier
 * that nothing arrives on.  The wait must run out, the kernel must return normally and leave the
 * wait-limit bit (8) in the device status word, which the next ss_device_status reports (SS_E_DEVICE)
 * and clears; the context stays usable.  *elapsed_ns = how long the kernel actually waited.
 * Synchronises the device. */
int ss_micro_wait_limit(int64_t limit_ns, int64_t* elapsed_ns);

/* Diagnostic.  No counterpart in the reference.  Runs one CTA that issues `iterations` x 2
 * back-to-back tcgen05.mma instructions of 128 channels x token_tile tokens (sparse kind::i8 with
 * K = 64 lifted columns, or dense kind::i8 with K = 32) on operands that rotate through shared
 * memory, optionally with the per-block metadata copy, and returns the cycles per instruction.
 * Used to show which resource bounds the GEMM main loop (shared-memory operand reads at
 * 128 B/clk/SM).  Synchronises the device; token_tile in {64, 128, 192, 256}. */
int ss_micro_mma_rate(int token_tile, int sparse, int with_metadata_copy, int iterations,
                      double* cycles_per_mma);

/* The complete projection (front-end + GEMM, no addend) for callers that cannot allocate device
 * memory at all: hosts whose HBM is fully carved into their own pools, loops in which
 * cudaMalloc/cudaFree are banned because they lock, block and may fail, plug-ins without access
 * to a framework allocator.  No counterpart in the reference, whose every entry allocates
 * through ATen.  The intermediate q/sa scratch that ss_projection takes from the caller lives in
 * a 32 MiB device array built into the library image (each GPU that loads the library holds it
 * until exit); the call allocates and frees nothing.  Limits and rules:
 *   - ceil32(m)*pk + ceil256(4*ceil32(m)) must be <= 32 MiB (33554432 bytes), else SS_E_LIMIT
 *     (1536 tokens x 18432 lifted columns fit; 4096 x 18432 do not);
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call before any
 *     stream capture begins;
 *   - "allocates nothing" holds from the second call on: with CUDA's lazy module loading the
 *     driver places the 32 MiB array and the two kernel images on the device when they are first
 *     used.  A host that carves up all of HBM should therefore make one warm-up call per device and
 *     per mode (or load with CUDA_MODULE_LOADING=EAGER) BEFORE it takes the memory, or that first
 *     call can fail with SS_E_CUDA;
 *   - all calls on a device share the one array: two calls whose kernels may overlap on the
 *     GPU (different streams, or graphs launched concurrently) race on it -- serialise them;
 *   - the array keeps the previous call's contents; nothing needs clearing because the
 *     front-end rewrites every byte the GEMM of the same call reads.
 * Arguments as ss_projection (inputs and outputs still belong to the caller). */
int ss_projection_static(const void* x_bf16, int64_t x_row_stride, int64_t m, int64_t k, int group,
                         const int8_t* packed, const int32_t* meta_b200,
                         const float* sw, const float* bias,
                         int64_t n, int64_t pn,
                         void* out_bf16, int64_t out_row_stride, void* stream);

/* ---- prepared plans (resident scratch; tensor maps come from the library's descriptor cache,
 *      so a plan's weights and resident scratch are encoded once) ----------------------------- */

/* Creates a plan for a fixed (m,k,n,group) on the current device; allocates its resident
 * q/sa scratch with cudaMalloc (the only allocating entry besides ss_plan_release's free).
 * Weight/scale/bias pointers are re-read at every run, so callers may overwrite their contents.
 * Returns 0 and the handle in *handle.  csrc/graph_projection.cuh:127-152 (prepare*). */
int ss_plan_create(const int8_t* packed, const int32_t* meta_b200, const float* sw,
                   const float* bias, int64_t k, int64_t m, int64_t n, int64_t pn, int group,
                   int64_t* handle);

/* Runs a plan.  On the stream that ran the plan last it uses the resident scratch; on another
 * stream, or while that stream is being captured into a CUDA graph, the caller must pass
 * scratch (q_scratch, sa_scratch) of the plan's size, else SS_E_ARG.
 * csrc/graph_projection.cuh:92-125,153-158 (Plan::forward, run). */
int ss_plan_run(int64_t handle, const void* x_bf16, int64_t x_row_stride,
                int8_t* q_scratch, float* sa_scratch,
                void* out_bf16, int64_t out_row_stride, void* stream);

/* Synchronises the plan's last stream and frees its scratch; unknown handles are ignored.
 * csrc/graph_projection.cuh:159-163 (release). */
int ss_plan_release(int64_t handle);

/* out[0..7] = {threads, dynamic smem bytes, registers, local bytes, CTAs/SM, token tile,
 * smem stages, TMEM columns}.  csrc/graph_projection.cuh:85-89,176 (resources). */
int ss_plan_resources(int64_t handle, int64_t* out, int n_out);

/* Resources of the GEMM kernel that a problem of this size would use (no plan needed); same
 * eight values as ss_plan_resources.  csrc/dualscale_sm80.cu:282-291 (configure_t). */
int ss_gemm_resources(int64_t m, int64_t n, int64_t pk, int64_t* out, int n_out);

/* ---- device status ------------------------------------------------------------------------ */

/* Synchronises `stream`, writes the device status word of the current device to *status and
 * clears it.  0 = no kernel gave up on a bounded wait since the last read: returns SS_OK.
 * Otherwise returns SS_E_DEVICE (bits: 1 TMA producer, 2 MMA issuer, 4 epilogue, 8 wait-limit
 * probe); outputs of the launches since the previous check are then not to be trusted (the call
 * also clears the sums a split-schedule launch may have left half done). */
int ss_device_status(void* stream, int32_t* status);

/* ---- tuning switches ----------------------------------------------------------------------- */

/* The library reads its switches from the environment once, at first use (SS_TOKEN_TILE,
 * SS_WIDE_CP, SS_META_WARP, SS_STORE, SS_RESIDENT, SS_PDL, SS_SPLIT, SS_WAIT_NS); these two entries read and
 * change them afterwards, for tests and measurements.  No counterpart in the reference.  Names:
 * "token_tile" (0 = automatic, or 128/192/224/240/256), "wide_cp", "meta_warp" (-1 = automatic),
 * "store" (1 = TMA-store epilogue), "resident" (weights-resident form), "pdl" (programmatic
 * dependent launch), "split" (schedule of the GEMM in which the clusters share the tiles x stages
 * evenly and a tile computed by several clusters is summed through device memory the library
 * allocates on the first such launch outside a stream capture, 152 MB (four areas of 38 MB, one per
 * stream that launches this schedule; further streams keep whole tiles): -1 = where the cost model prefers it, 0 never,
 * 1 wherever the output form allows; the results are the same bits either way), "wait_ns" (limit
 * of every device-side wait, default 2e9).  ss_get_option also answers "split_launches": how many
 * GEMM launches of this process took the split schedule.  Not synchronised with concurrent
 * launches from other threads. */
int ss_set_option(const char* name, int64_t value);
int ss_get_option(const char* name, int64_t* value);

#ifdef __cplusplus
}
#endif
#endif /* SLIDESPARSE_B200_H */
