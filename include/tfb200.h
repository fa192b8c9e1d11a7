/* tfb200.h - C ABI of the B200 (sm_100a) routed-expert MoE library, libtfb200.so.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (cudaStream_t passed as void*), enqueues its
 * work on that stream for the CURRENT device, never synchronises the host and never allocates.  The return value is a
 * status: 0 ok; -1 a bad argument (nothing was launched); -2 the CUDA runtime refused a call; the text is available
 * from tfb_last_error() on the calling thread.  Grids are sized by host-known upper bounds and the true counts are read
 * on the device, so a captured CUDA graph follows new routing on replay.
 *
 * Each declaration names the interface of the reference (bertholomus/TensorFold, paths inside its tree) it replaces.
 * bf16 / fp16 buffers are passed as const void*; int32 buffers as int32_t*.
 */
#ifndef TFB200_H
#define TFB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library state ------------------------------------------------------------------------------------------- */

/* Text of the calling thread's last failure (never NULL). */
const char* tfb_last_error(void);

/* ABI version of this header (1). */
int tfb_version(void);

/* Launch with programmatic stream serialization (kernels overlap their prologue with the previous kernel's tail and
 * wait on the device before touching memory).  Returns the previous setting.  Off by default. */
int tfb_set_pdl(int on);

/* Reads and clears the current device's status word into *status; synchronises `stream`.  0: every bounded wait
 * completed.  Otherwise code | where << 8 | rank << 16: code 1 = a bounded wait ran out and the kernel returned early,
 * 2 = a table held an index no kernel exists for; where (code 1) 0 = a kernel's own copy pipeline, 1 = the tokens
 * barrier of an expert-parallel step, 2 = its results barrier; rank (where 1, 2) = the lowest rank that had not
 * arrived.  After a barrier time-out the kernels of that step leave the peers' memory alone and its output is void.
 * The trap's counterpart (src/tensorfold/cuda/exl3/experts_grouped.cuh:240,259) and, for the barriers, the named
 * missing rank of NCCL.ready (src/tensorfold/cuda/comm.py:78-101). */
int tfb_kernel_status(int* status, void* stream);

/* Milliseconds an expert-parallel barrier waits for the other ranks before it gives up (1 .. 600000; 1000 unless
 * set); returns the previous limit, or -1 with a message.  Read at launch (and at graph capture).  Counterpart of the
 * `timeout` of NCCL.ready (src/tensorfold/cuda/comm.py:78). */
int tfb_set_wait_limit_ms(int ms);

/* ---- routing ------------------------------------------------------------------------------------------------- */

/* logits[T, NE] fp32 = x[T, D] (bf16, row stride x_stride elements) . rows[NE, D]^T (bf16), fixed summation order.
 * Replaces moe.router / the Triton kernel _router: src/tensorfold/cuda/moe.py:23-55. */
int tfb_router(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE, void* stream);

/* The same logits for prompts, on the tensor cores (bf16 mma, fp32 accumulate, a fixed summation order of its own: the
 * last bits differ from tfb_router's; a row's bits do not depend on the call's other rows).  D a multiple of 32.
 * The reference's router changes its blocking with the row count in the same way: src/tensorfold/cuda/moe.py:23-55. */
int tfb_router_prompt(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE,
                      void* stream);

/* Per row: the top_k experts among the first E logits (largest first, ties to the lower id), weights
 * bf16(exp(l_k - l_0) / sum) stored as fp32; when `shared` != 0 one more slot holds id E with weight
 * bf16(sigmoid(bf16(logits[r, E]))).  pick / wts are [T, top_k + (shared != 0)], NL is the logits' row length.
 * Replaces moe.select_rows / _topk_rows: src/tensorfold/cuda/moe.py:58-85,103-108. */
int tfb_select_rows(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k, int shared,
                    void* stream);

/* Sigmoid-plus-bias routers: score = sigmoid(logit); the top_k experts by score + bias[e] (ties to the lower id);
 * weights = the picked scores, over their sum in pick order (+ 1e-20) when norm, times scale; then shared_slots slots
 * with ids E, E + 1, .. and weight 1.  pick / wts are [T, top_k + shared_slots].
 * Replaces _topk / select: src/tensorfold/families/glm5_next/cuda/glue.py:351-390 (one shared slot) and _topk of
 * src/tensorfold/families/nemotron_h/cuda/glue.py:50-100 (two shared halves). */
int tfb_select_sigmoid(const float* logits, int NL, const float* bias, int32_t* pick, float* wts, int T, int E,
                       int top_k, int shared_slots, float scale, int norm, void* stream);

/* Groups the pairs p = row * slots + slot by ascending expert, pair order kept inside an expert: members[pairs],
 * items[n, 3] = (expert, first member, count <= tile) in expert order then chunk order, counts = (items, distinct
 * experts).  Ids outside [0, experts) are left out.  experts <= 1024.  One launch at any pair count.
 * Replaces the extension entry `plan`: src/tensorfold/cuda/experts.cpp:33-41, experts.cu:157-334 (its rank / hist
 * scratch is not needed). */
int tfb_plan(const int32_t* picks, int64_t pairs, int experts, int tile, int32_t* members, int32_t* items,
             int32_t* counts, void* stream);

/* tfb_select_rows followed by tfb_plan in ONE launch (one thread block) for calls of at most
 * tfb_select_plan_max_rows() rows: same pick / wts / members / items / counts, bit for bit.  The plan covers
 * E + (shared != 0) experts.  Replaces moe.select for decode-sized calls: src/tensorfold/cuda/moe.py:111-116. */
int tfb_select_plan_max_rows(void);
int tfb_select_plan(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k, int shared,
                    int tile, int32_t* members, int32_t* items, int32_t* counts, void* stream);

/* Expert-parallel forms (no reference counterpart: the reference has no expert parallelism, src/tensorfold/cuda/comm.py
 * is an all-gather for 2-rank tensor parallelism).  A "window" is the contiguous id range [lo, lo + n) of the experts a
 * rank owns; plans are made over those ids renumbered from 0, and tfb_combine_window sums only those slots. */
int tfb_plan_window(const int32_t* picks, int64_t pairs, int lo, int experts, int tile, int32_t* members,
                    int32_t* items, int32_t* counts, void* stream);
/* tfb_plan_window with the busy experts set apart: experts with at least `hot` pairs get their items (of up to
 * big_tile pairs) in big_items / big_counts, for tfb_experts_prefill; the rest stay in items / counts (of up to `tile`
 * pairs), for tfb_experts_run.  Both tables index the one members array.  No reference counterpart. */
int tfb_plan_split(const int32_t* picks, int64_t pairs, int lo, int experts, int tile, int big_tile, int hot,
                   int32_t* members, int32_t* items, int32_t* counts, int32_t* big_items, int32_t* big_counts,
                   void* stream);
int tfb_select_plan_window(const float* logits, int NL, int32_t* pick, float* wts, int T, int E, int top_k, int shared,
                           int tile, int plan_lo, int plan_n, int32_t* members, int32_t* items, int32_t* counts,
                           void* stream);

/* tfb_router, tfb_select_rows and tfb_plan_window of a few rows in ONE launch, with the same bits: logits [T, NE] fp32
 * from x [T, D] and rows [NE, D] (NE = E + 1 with the shared expert's gate row), pick / wts [T, slots], and the plan of
 * the ids in [plan_lo, plan_lo + plan_n).  The CTA that finishes a group of eight rows selects them; the one that
 * finishes the last group plans.  arrive: int32 scratch [1 + (T + 7) / 8], zero before the first call (a call leaves it
 * zero).  T <= tfb_route_max_rows(NE).  Replaces the three launches of moe.moe's routing:
 * src/tensorfold/cuda/moe.py:41-55,103-116 and src/tensorfold/cuda/experts.py:101-125. */
int tfb_route_max_rows(int NE);
int tfb_route(const void* x, int64_t x_stride, const void* rows, float* logits, int T, int D, int NE, int E, int top_k,
              int shared, int32_t* pick, float* wts, int tile, int plan_lo, int plan_n, int32_t* members,
              int32_t* items, int32_t* counts, int32_t* arrive, void* stream);
int tfb_combine_window(const void* y, int y_bf16, const float* wts, const int32_t* pick, int lo, int n, void* out,
                       int out_f32, int T, int slots, int D, void* stream);

/* The combine, the residual add and the RMSNorm behind a MoE block in one pass over each row: delta = bf16(sum over
 * the first `routed` slots of wt * y, an fp32 fma chain in slot order, + the other (shared) slots' y); hn = bf16(h +
 * delta); out = bf16(hn * rsqrt(mean(hn^2) + eps) * w); xs [R, D / 64] fp32 = the sums of out over groups of 64 (what
 * the next 4-bit projection wants).  y [R, slots, D] fp32, or bf16 when y_bf16; D a multiple of 64, at most 8192.
 * Replaces `add_moe_norm`: src/tensorfold/families/nemotron_h/cuda/glue.py:104-141. */
int tfb_add_moe_norm(const void* h, const void* y, int y_bf16, const float* wt, const void* w, void* hn, void* out,
                     float* xs, int R, int D, int slots, int routed, float eps, void* stream);

/* Expert parallelism over NVLink peer memory (no reference counterpart, as above): the token exchange and the return of
 * the results done by this library's kernels with plain loads and stores to the peers' windows, no collective library
 * on the path.  `windows` is a DEVICE array of `world` pointers: entry i is rank i's window as mapped into this process
 * (entry `rank` is this rank's own memory).  A window holds [2][world] uint32 barrier flags (zero at start), the regions
 * the peers pull (the rank's tokens; its rows' experts and weights) and the result buffer of world * rows_local * D * 4
 * bytes at p_offset.  `step` is one uint32 in device memory, zero at start, counted up by tfb_combine_push.  One step,
 * the same on every rank:
 *   [tfb_peer_stage, or the caller writes its tokens into the window]  router and selection of the rank's own rows,
 *   written into the window   tfb_peer_gather (tokens barrier, then pull)   plan of the rank's experts   gate/up
 *   down   tfb_combine_push   tfb_peer_sum (results barrier, then sum in rank order).
 * A barrier's wait gives up after tfb_set_wait_limit_ms and records the barrier and the missing rank in the device
 * status word; from then on the step's kernels touch no peer memory.  Read tfb_kernel_status after a step before its
 * output is used.  A barrier needs every rank's kernel to be running at the same time, so the ranks must be separate
 * GPUs. */
int tfb_peer_stage(const void* x_local, void* window, int64_t x_offset, int64_t x_bytes, void* stream);
/* nseg <= 4 regions (host arrays): seg_dst[s][r * seg_bytes[s] ...] <- rank r's window + seg_offset[s], every r. */
int tfb_peer_gather(void* const* windows, int rank, int world, int nseg, const int64_t* seg_offset,
                    const int64_t* seg_bytes, void* const* seg_dst, const void* step, void* stream);
/* tfb_combine_window with fp32 output, each token's row stored into its home rank's result buffer, slot `rank`. */
int tfb_combine_push(const float* y, const float* wts, const int32_t* pick, int lo, int n, void* const* windows,
                     int64_t p_offset, int rank, int rows_local, int T, int slots, int D, void* step, void* stream);
/* The same hand-over for partial sums another kernel formed: row r of partial [T, D] fp32 goes to its home rank. */
int tfb_peer_push(const float* partial, void* const* windows, int64_t p_offset, int rank, int rows_local, int T, int D,
                  void* step, void* stream);
/* Selections as the owner of experts [lo, lo + n) sees them: its ids renumbered from 0 with their weights, every other
 * slot as id n (skipped by the expert kernels) with weight 0. */
int tfb_window_picks(const int32_t* pick, const float* wts, int lo, int n, int32_t* pick_out, float* wts_out,
                     int count, void* stream);
/* out[rows_local, D] (bf16, or fp32 with out_f32) = the ranks' partial sums added in rank order, then, when given,
 * extra_w[j * extra_w_stride] * extra[j, :] (the replicated shared expert of the rank's own rows), then, when given,
 * the residual rows [rows_local, D] bf16 (the layer's input: out = h + layer(h) with no pass of its own; not the same
 * memory as out); rounded once. */
int tfb_peer_sum(void* const* windows, int rank, int64_t p_offset, int world, int rows_local, int D, void* out,
                 int out_f32, const float* extra, const float* extra_w, int extra_w_stride, const void* residual,
                 const void* step, void* stream);

/* out[T, D] = sum over slots, in slot order, of wts[T, slots] * y[T, slots, D] (fp32 fma chain from 0), rounded once.
 * y is fp32 (y_bf16 = 0) or bf16; out is bf16 (out_f32 = 0) or fp32.
 * Replaces moe.combine / _combine: src/tensorfold/cuda/moe.py:131-151, and combine_kernel of
 * src/tensorfold/cuda/exl3/experts.cu:181-190 for the fp32 form. */
int tfb_combine(const void* y, int y_bf16, const float* wts, void* out, int out_f32, int T, int slots, int D,
                void* stream);

/* xs[M, K/gs] fp32 = the sum of each group of gs = 64 inputs of x[M, K] bf16 (row stride x_stride elements).
 * Replaces group_sums / _group_sums: src/tensorfold/cuda/kernels/qmm.py:137-153. */
int tfb_group_sums(const void* x, int64_t x_stride, float* xs, int M, int K, int gs, void* stream);

/* ---- MLX affine 4-bit group-64 experts -------------------------------------------------------------------------- */

/* words [E, N, K/8] (uint32, element k of a row at bits 4 (k % 8) of word k / 8), scales and biases [E, N, K/gs]
 * (2-byte: bf16 or fp16, carried opaquely) -> out int32 [E, N/32, K/gs, 288].  gs must be 64.
 * Replaces the extension entry `pack`: src/tensorfold/cuda/experts.cpp:58-75, experts_pack.cu. */
int tfb_pack(const void* words, const void* scales, const void* biases, int gs, void* out, int E, int N, int K,
             void* stream);

/* pack's inverse on the device (the reference's is torch indexing: src/tensorfold/cuda/experts.py:43-58). */
int tfb_unpack(const void* blocks, int gs, void* words, void* scales, void* biases, int E, int N, int K, void* stream);

/* The weight values the kernels multiply by, out [E, N, K]: mode 0 fp32 fma(scale, q, bias) (decode form); mode 1 the
 * prefill form's bf16 weights.  sb_type 0: bf16 scales, 1: fp16 scales.  The hook for the bit-exactness checks
 * (the reference's twins: src/tensorfold/families/qwen3_5_moe/cuda/weights.py:20-29,
 * src/tensorfold/cuda/experts_prefill.cu:25-29). */
int tfb_dequant(const void* blocks, int gs, int sb_type, int mode, void* out, int E, int N, int K, void* stream);

/* Grouped 4-bit expert matmul, decode form, over a plan.  x: bf16 rows of K = kg * gs inputs (row stride x_stride
 * elements, 16-byte aligned); pair p reads row p / slots when slots > 0, else row p.  w: blocks
 * [E, nb, kg, M, 288] (M = 2 for epi 2, else 1).  out rows of n = 32 * nb columns, row index = pair id.
 * Items hold at most 8 pairs in this form (plan with tile 8).
 * epi 0: fp32 out; 1: bf16 relu(bf16 acc)^2; 2: bf16 SwiGLU(matrix 0, matrix 1) clipped at `limit` when > 0;
 * 3: bf16 out.  max_units = upper bound of items * nb (the grid); the items table must hold that many items (rows
 * past counts[0] are read, not used).  sb_type as tfb_dequant.
 * Replaces the extension entry `run`: src/tensorfold/cuda/experts.cpp:43-48, experts.cu:130-155,287-351. */
int tfb_experts_run(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                    const int32_t* items, const int32_t* counts, const int32_t* members, void* out, int n, float limit,
                    int64_t max_units, int sb_type, void* stream);

/* tfb_experts_run over a plan whose items hold up to `tile` = 8 or 16 pairs.  With 16 every weight fragment is
 * dequantised once for two mma tiles of pairs (worth it from about 9 pairs an expert); a pair's bits do not depend on
 * the tile.  No reference counterpart (its decode items always hold 16: src/tensorfold/cuda/experts.py:13). */
int tfb_experts_run_tile(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                         const int32_t* items, const int32_t* counts, const int32_t* members, void* out, int n,
                         float limit, int64_t max_units, int sb_type, int tile, void* stream);

/* The decode form with its K slices left apart: part [tfb_decode_kslices(kg), rows, n] fp32, slice k of pair p at
 * part[k, p, :]; adding the slices in order k = 0, 1, .. gives epilogue 0's bits.  For a caller that folds the sum into
 * its next kernel.  Replaces `matmul(reduce=False, part=)`: src/tensorfold/cuda/kernels/qmm.py:156-177. */
int tfb_experts_run_slices(int gs, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                           const int32_t* items, const int32_t* counts, const int32_t* members, float* part, int n,
                           int rows, int64_t max_units, int sb_type, int tile, void* stream);

/* K slices the decode form cuts a projection of kg groups of 64 inputs into: a function of the shape alone. */
int tfb_decode_kslices(int kg);

/* The down projection and the weighted combine in one launch: y [P, n] fp32 per pair exactly as tfb_experts_run_tile
 * with epilogue 0 (x = act [P, K] bf16, one row a pair), and out [T, n] (bf16, or fp32 when out_f32) = the sum over a
 * token's slots in slot order of wts[t, s] * y[t * slots + s, :] (an fp32 fma chain from 0, rounded once), formed by
 * the CTA that stores the token's last row.  Every pair t * slots + s of the call's tokens must be in the plan.
 * arrive: int32 scratch [T, nb], zero before the first call (a call leaves it zero).
 * Replaces `down` followed by `combine`: src/tensorfold/cuda/experts.py:141-150, src/tensorfold/cuda/moe.py:131-151. */
int tfb_experts_down_combine(int gs, const void* x, int64_t x_stride, const void* w, int kg, int nb,
                             const int32_t* items, const int32_t* counts, const int32_t* members, float* y, int n,
                             int64_t max_units, int sb_type, int tile, const float* wts, int slots, void* out,
                             int out_f32, int32_t* arrive, void* stream);

/* Grouped 4-bit expert matmul, prefill form (tcgen05 tensor cores, weights dequantised to bf16 with one rounding,
 * one fp32 chain over K).  Arguments as tfb_experts_run, but items may hold up to 192 pairs (plan with tile <= 192) and
 * max_items = an upper bound of the item count.
 * Replaces the extension entry `prefill`: src/tensorfold/cuda/experts.cpp:50-56, experts_prefill.cu:31-195. */
int tfb_experts_prefill(int gs, int epi, const void* x, int64_t x_stride, int slots, const void* w, int kg, int nb,
                        const int32_t* items, const int32_t* counts, const int32_t* members, void* out, int n,
                        float limit, int64_t max_items, int sb_type, void* stream);

/* ---- EXL3 trellis-coded experts ------------------------------------------------------------------------------- */
/* Trellises are int16 [K/16, N/16, 8 * k2] (k2 = half-bits a value, 2..16), read in place; cb 0 = 3inst, 1 = mcg,
 * 2 = mul1; suh / svh are fp16 [E, n].  K and N are multiples of 128. */

/* W_q [K, N] fp16 of one trellis through the kernels' lane decode (the bit-exactness hook).
 * Replaces `dequant`: src/tensorfold/cuda/exl3/experts.cpp:132-141, experts_grouped.cuh:287-306. */
int tfb_exl3_dequant(const void* trellis, void* out, int K, int N, int k2, int cb, void* stream);

/* pick [R, slots] -> uids [maxu] = the distinct routed experts (< E) ascending, ucount [1], members [maxu, maxm] =
 * row * 32 + slot in row order, -1 after the last.  members must hold maxu * maxm words: only the rows of the
 * ucount experts found are written, experts past maxu are left out and an expert's members past maxm are cut off
 * (maxu >= min(R * slots, E) and maxm >= R lose nothing).  tmp_members [R * slots], tmp_items [3 * min(R * slots, E)]
 * and tmp_counts [2] are caller scratch.  E <= 1024, slots <= 32.
 * Replaces `group`: src/tensorfold/cuda/exl3/experts.cu:19-72,290-310. */
int tfb_exl3_group(const int32_t* pick, int32_t* uids, int32_t* ucount, int32_t* members, int32_t* tmp_members,
                   int32_t* tmp_items, int32_t* tmp_counts, int R, int slots, int E, int maxu, int maxm, void* stream);

/* tfb_exl3_group without the three scratch arguments: the sort's temporaries sit in an array built into the library
 * (about 140 KB on every GPU that loads it).  No counterpart in the reference; it exists for hosts that cannot allocate
 * device memory when they call (all HBM already given to their own pools, or allocation calls banned on the decode
 * path because they stall the device).  Limits: R * slots <= 32768 pairs, E <= 1024, slots <= 32; larger calls are
 * refused with an error naming tfb_exl3_group.  The first call on a device resolves the array's address - make it
 * before any stream capture begins.  Calls on one GPU share the array: do not let two run concurrently. */
int tfb_exl3_group_static(const int32_t* pick, int32_t* uids, int32_t* ucount, int32_t* members, int R, int slots,
                          int E, int maxu, int maxm, void* stream);

/* The first launch of a routed EXL3 call.  When `sort` != 0 (then 16 or 32: the pairs an item holds) one block sorts
 * the (row, slot) pairs by expert: members [R * slots] = pair ids grouped by ascending expert (pair order kept),
 * items [., 3] = (expert, first, count <= sort) with room for min(R * slots, E) + R * slots / sort rows, counts [2] =
 * (items, distinct experts),
 * ucount [1] = distinct experts; ids outside [0, E) are left out.  The other blocks rotate the inputs:
 * out0 / out1 [R * slots, K] fp16 = fp16(((x * suh_m[expert]) H) / sqrt(128)) for the two matrices of every routed pair
 * (suh1 and out1 null: one matrix); x is bf16 (x_is_fp16 = 0) or fp16 rows with stride x_stride.
 * sorted (or null; needs `sort`): int32 [3, sorted_stride, 4], 16-byte aligned, filled with the items as (expert,
 * first, count, index) once in the order of each projection's widths k2_g / k2_u / k2_d [E], widest first - hand the
 * three tables to tfb_exl3_gateup / tfb_exl3_down when a layer's tensors differ in width, so that blocks that run
 * together decode one width; sorted_stride >= the sort's item count.
 * Replaces `group` and `rot_in`: src/tensorfold/cuda/exl3/experts.cu:19-111,290-330. */
int tfb_exl3_prologue(const void* x, int64_t x_stride, int x_is_fp16, const int32_t* pick, const void* suh0,
                      const void* suh1, void* out0, void* out1, int R, int K, int slots, int E, int sort,
                      int32_t* members, int32_t* items, int32_t* counts, int32_t* ucount, const int32_t* k2_g,
                      const int32_t* k2_u, const int32_t* k2_d, int32_t* sorted, int sorted_stride, void* stream);

/* xd [P, N] fp16 = the down projection's rotated input of every routed pair, in one launch: gate and up (xg, xu
 * [P, K] fp16 times W_q of each pair's expert, trellises decoded on the fly from 16-byte aligned tp_* [E] at widths
 * k2_* [E]), output rotation, svh, SwiGLU (act_mode 0: bf16 roundings, 1: fp32; clipped at limit), suh_d, rotation.
 * items / counts / members: the prologue's sort; z: fp32 scratch [2, P, N]; arrive: int32 scratch
 * [max_items * N / 128], zero before the first call (a call leaves it zero); max_items >= the sort's item count.
 * sorted_g / sorted_u (both or neither): the prologue's width-ordered items of the two matrices, [., 4] each.
 * item_pairs: 16 or 32, the most pairs an item holds (with 32 one decode of a weight tile serves up to 32 pairs, at
 * more registers a thread: for calls with many pairs an expert); a pair's bits do not depend on it.
 * k2_all: 0, or the width every entry of k2_g and k2_u has - a promise that lets the launch use a kernel built for
 * that width alone (a tenth of the code; it pays at a few tokens); a tensor of another width then sets the status
 * word and nothing is stored.  -1: the widths differ - the launch uses a build with short loops, so that blocks
 * decoding different widths share an SM's instruction cache (col_tiles 4).  col_tiles: 4 or 2, the 16-column tiles a thread block takes (2 doubles the blocks of
 * a launch that would otherwise leave SMs idle: few experts in use; offered with k2_all = 8 only); no result depends
 * on it.
 * Replaces `grouped` + `gateup_epilogue`: src/tensorfold/cuda/exl3/experts_grouped.cuh:190-284,
 * src/tensorfold/cuda/exl3/experts.cu:116-158. */
int tfb_exl3_gateup(const void* xg, const void* xu, const int64_t* tp_g, const int64_t* tp_u, const int32_t* k2_g,
                    const int32_t* k2_u, const int32_t* items, const int32_t* counts, const int32_t* members, float* z,
                    int32_t* arrive, const void* svh_g, const void* svh_u, const void* suh_d, void* xd, int K, int N,
                    int P, int cb, int max_items, float limit, int act_mode, const int32_t* sorted_g,
                    const int32_t* sorted_u, int item_pairs, int k2_all, int col_tiles, void* stream);

/* y [P, N] fp32 = rotate(x [P, K] fp16 times W_q of each pair's expert) * svh for every routed pair (other rows are
 * left as they are), in one launch; z: fp32 scratch [P, N]; the other arguments as tfb_exl3_gateup (sorted: the
 * prologue's width-ordered items of the down matrices, or null; k2_all: 0 or the one width of every k2 entry; col_tiles as there).  The weighted
 * slot-order sum over a row's slots is tfb_combine on y.
 * Replaces `grouped` + `down_epilogue` (+ `combine`, `down_combine`): src/tensorfold/cuda/exl3/experts.cu:161-237. */
int tfb_exl3_down(const void* x, const int64_t* tp, const int32_t* k2, const int32_t* items, const int32_t* counts,
                  const int32_t* members, float* z, int32_t* arrive, const void* svh, float* y, int K, int N, int P,
                  int cb, int max_items, const int32_t* sorted, int item_pairs, int k2_all, int col_tiles,
                  void* stream);

/* The output side of an EXL3 product formed elsewhere (prompts: a dense fp16 GEMM over the decoded W_q):
 * out [M, N] (out_type 0 fp32, 1 fp16, 2 bf16; rows out_stride elements apart) = rotate(z) / sqrt(128) * svh + bias
 * for every 128-column block of z [M, N] fp32; bias fp16 [N] or null.
 * Replaces the epilogue of `_gemm`: src/tensorfold/cuda/exl3/prefill.py:15-44. */
int tfb_exl3_rot_out(const float* z, const void* svh, const void* bias, void* out, int64_t out_stride, int out_type,
                     int M, int N, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TFB200_H */
