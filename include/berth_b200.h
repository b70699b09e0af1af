/*
 * berth_b200.h -- C ABI of libberth_b200.so: the EXL3 trellis-linear / A3B-MoE hot path of
 * berth, written for NVIDIA B200 (sm_100a).
 *
 * Conventions, identical to the library berth's Rust crate `berth-kernels` binds
 * (crates/berth-kernels/src/ffi.rs:1-24, src/prefill_lin.rs:33-80, src/ops.rs:13-148):
 *   - every tensor pointer is a DEVICE address; the caller owns the buffers and keeps them
 *     alive until `stream` has finished; `stream` is a cudaStream_t, NULL = default stream;
 *   - launches are asynchronous on `stream`; nothing here synchronises the device;
 *   - return 0 = ok, -1 = error (berth_ops_mgemm: > 0 = ok, <= 0 = error); no C++ exception
 *     crosses the boundary; the message of the last failed call and the description of the
 *     last successful launch are kept per host thread and stay valid until the next call of
 *     the same family on that thread;
 *   - host checks (null pointer, size, bitrate, codebook) fail before any CUDA call, with the
 *     substrings berth's tests look for: "null", "positive", "multiple of 16",
 *     "multiple of 128", "size_m", "no linked kernel";
 *   - an unsupported shape fails closed; there is no fallback kernel, no CPU path, no
 *     runtime autotuning, no environment-variable policy and no file written anywhere.
 *
 * Tensor layout (crates/berth-kernels/src/lib.rs:86-103):
 *   a        fp16 [size_m][size_k]                     activations, row major
 *   trellis  int16 [size_k/16][size_n/16][16*k_bits]   one 16x16 weight tile per last-dim row
 *   suh      fp16 [size_k]   input-side sign-scale;  svh fp16 [size_n] output-side sign-scale
 *   a_had    fp16 [size_m][size_k]   scratch the kernel fills with H128(a*suh)/sqrt(128)
 *   c        fp16 or fp32 [size_m][size_n]
 *   codebook 0 = 3INST, 1 = MCG, 2 = MUL1 (crates/berth-kernels/src/lib.rs:49-63)
 *
 * Per-device state owned by the library, allocated at the first launch on a device and kept
 * until exit (the counterpart of the lock buffer and 16 MiB split-K workspace of
 * crates/berth-kernels/csrc/linear.cu:334-345 and csrc/int8_sq.cu:20-47): about 40 MiB (split-K
 * partial-sum slabs, rotated activations, block sums).  Launches of the decode kernels (up to 32
 * rows, and the grouped decode launches of the MoE layer) that overlap on one device (different
 * streams) must not share it: berth drives one stream per device, and so must every other caller.
 * The prefill kernels use none of it.  The kernels of one linear are chained by programmatic
 * dependent launch: a decode kernel may prefetch weights while the kernel before it on the stream
 * still runs, so the trellis must not be written by the kernel that directly precedes a linear.
 */
#ifndef BERTH_B200_H
#define BERTH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ decode linear (m >= 1)
 * Replaces berth_exl3_linear (crates/berth-kernels/src/ffi.rs:7-21,
 * crates/berth-kernels/csrc/linear.cu:209-286,362-394): c = H(H(a*suh) . W(trellis)) * svh.
 * Serves every size_m: one row of a MUL1 matrix on the integer-path decode kernel (codebook byte sums in tensor
 * memory, tcgen05.mma kind::i8, rotation and finishing inside the kernel); up to 16 rows (and up to 32 of a small
 * matrix) the fused decode GEMV; 17..32 rows of a large matrix the persistent split-K tensor-core kernel; above, the
 * tiled tcgen05 tensor-core GEMM.  berth_exl3_last_launch names the kernels that ran.  Programmatic-launch contract:
 * the kernels start fetching `trellis` while the kernel before them on the stream may still be running, so the
 * weights must be final before that kernel starts; every other tensor is touched only after the predecessor ended. */
int berth_exl3_linear(const void* a, const void* trellis, void* c, const void* suh, void* a_had,
                      const void* svh, int size_m, int size_k, int size_n, int k_bits,
                      int codebook, int out_fp32, void* stream);
const char* berth_exl3_last_error(void);    /* crates/berth-kernels/csrc/linear.cu:396-399 */
const char* berth_exl3_last_launch(void);   /* crates/berth-kernels/csrc/linear.cu:401-404 */

/* Same linear for callers that must not allocate device memory (a host whose own planner owns
 * every byte of HBM, or a decode loop that cannot take cudaMalloc's device-wide synchronisation).
 * No counterpart in berth: its library allocates its workspaces with cudaMalloc at first use.
 * The scratch is a fixed __device__ array of about 6.2 MiB inside the library image (4 MiB
 * partial-sum slabs, 2 MiB rotated activations, 128 KiB block sums, 16 KiB counters, a status word),
 * held by every GPU that loads the library until the process exits; nothing is allocated or freed.
 * Limits: size_m <= 32, size_n <= 131072 and size_k * g <= 131072 with g = 1, 2, 4 for up to 8, 16, 32
 * rows; larger sizes are rejected with an error before anything is launched.  With 17..32 rows the slab
 * area holds the partial sums of 64 CTAs, so those launches run on 64 SMs.  The first
 * call on a device looks the array's device address up (cudaGetSymbolAddress); make that first
 * call before any stream capture begins.  All calls on a device share the scratch, which keeps
 * the previous call's contents (every part is overwritten before it is read): calls that overlap
 * on the GPU race, so issue them on one stream. */
int berth_exl3_linear_static_scratch(const void* a, const void* trellis, void* c, const void* suh,
                                     void* a_had, const void* svh, int size_m, int size_k,
                                     int size_n, int k_bits, int codebook, int out_fp32,
                                     void* stream);

/* Guard for the programmatic-launch contract above.  By default the decode kernels start fetching `trellis` while the
 * kernel before them on the stream may still be running.  A host that writes weights on the same stream directly before
 * the linear that reads them (experts or layers streamed in) calls berth_exl3_weights_streamed(1) once: from then on no
 * kernel of this process fetches weights before its predecessor has ended -- berth's own rule (stream order is enough,
 * crates/berth-kernels/src/lib.rs:126-133) at the price of the overlap.  Returns the previous setting.  No CUDA call.
 * No counterpart in berth. */
int berth_exl3_weights_streamed(int on);

/* Device queries of crates/berth-kernels/csrc/internal.h:11-13 (class 1..5 as the fork's CC_*
 * enumeration orders them: old, Ampere, Ada, Hopper, Blackwell; SM count). -1 on error. */
int berth_device_cc(int device);
int berth_device_sms(int device);
/* Reads and clears the status words of the kernels on `device`: the library's workspace and the
 * fixed scratch of berth_exl3_linear_static_scratch, OR-ed together (this call synchronises the
 * device).  The kernels never wait without a limit: a wait that runs out sets a bit here and the
 * launch finishes with undefined output instead of hanging.  Bits: 1 = a weight stage never arrived,
 * 2 = a stage was never released, 4 = a tensor-memory stage or accumulator of the integer-path decode
 * kernel was never handed over, 16 = a wait of the tensor-core GEMM ran out, 32 = a peer's flag of the
 * expert-parallel exchange never arrived, 64 = rows did not fit a receive buffer or a problem table of
 * the expert stage.  0 = clean, -1 = CUDA error.  No counterpart in berth. */
int berth_device_status(int device);

/* Diagnostic, no counterpart in berth: the bare decode rate of one SM.  Runs the inner loop of the
 * decode GEMV (tile words in shared memory -> window extraction -> codebook arithmetic -> MMA) with
 * no global-memory traffic on every SM with `warps` warps for `iters` iterations of eight tiles per
 * warp, and returns the decoded weights per clock per SM (mean over the SMs) and the SM clock seen
 * during the run.  path 0 = fp16 tensor path (every codebook); MUL1 on the integer path: 1 = with the warp-level
 * mma.sync.m16n8k32, 2 = with the products stored to tensor memory as the decode kernel does (at most 16 warps).
 * k_bits 3..6.  Allocates three small buffers, synchronises the device, frees them. */
int berth_exl3_decode_rate(int k_bits, int codebook, int path, int warps, int iters,
                           double* weights_per_clk_sm, double* sm_mhz);
/* Diagnostic, no counterpart in berth: which instructions of the decode loop share an issue pipe.  16 warps per SM run a
 * bundle of independent instructions `iters` times; the result is the cycles one bundle costs a warp scheduler.
 * kind 0 = two mma.sync.m16n8k16 (fp16); 1 = those plus eight lop3; 2 = those plus eight 32-bit multiplies; 3 = eight
 * lop3 plus eight multiplies; 4 = two mma.sync.m16n8k32 (u8 x s8); 5 = those plus eight lop3. */
int berth_exl3_pipe_probe(int kind, int iters, double* clk_per_iteration_per_scheduler);

/* FNV-1a shape key of crates/berth-kernels/csrc/linear.cu:65-104,345-358.  Kept because berth's
 * tests pin its value; this library never tunes at run time.  No CUDA call. */
uint64_t berth_exl3_gemm_tune_key(int size_m, int size_k, int size_n, int k_bits, int out_fp32,
                                  int device, int cc, int sms, int cb);

/* Smallest-shape self tests of crates/berth-kernels/csrc/linear.cu:406-465 (allocate, launch,
 * synchronise, free).  0 = ok. */
int berth_exl3_smoke_int8(int out_fp32);
int berth_exl3_smoke_gemm(void);

/* The decode linear (size_m <= 32) with the greedy arg-max of every output row taken in the finishing step: what
 * berth does for the lm_head with the K = 6 linear (crates/berth-kernels/csrc/linear.cu:131-207) followed by the
 * two kernels of its fused sampler in greedy mode (crates/berth-kernels/csrc/sample/fused.cu:45-135, mode 0), in
 * the launches of the linear alone.  best: DEVICE array of size_m 64-bit keys (zeroed by the call on the stream);
 * after the stream completes key r describes the largest output of row r, ties to the lower column, the value as
 * stored (fp16-rounded for fp16 outputs); berth_argmax_key_decode splits a key on the host.  c may be NULL: the
 * outputs are then not written at all.  Everything else as berth_exl3_linear; the call always runs the decode
 * kernel, so from 17 rows of a large matrix (where berth_exl3_linear runs the split-K tensor-core kernel) its
 * outputs equal berth_exl3_linear's within the accumulation tolerance instead of bit for bit. */
int berth_exl3_linear_argmax(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                             unsigned long long* best, int size_m, int size_k, int size_n, int k_bits, int codebook,
                             int out_fp32, void* stream);
void berth_argmax_key_decode(unsigned long long key, int32_t* token, float* value);
/* The same with berth's fused sampler in either of the modes its serve launches (crates/berth-kernels/csrc/sample/
 * fused.cu:45-135: berth_sample_fused, mode 0 greedy, mode 1 Gumbel arg-max over logits * inv_temp) taken in the
 * finishing step of the linear.  mode 1: key r describes the column that maximises
 *   stored output[r][col] * inv_temp + g(random, r, col),   g = -log(-log(u)),
 * u = (k + 1/2) / 2^23 with k the upper 23 bits of a 32-bit mixing hash of (random, r, col) -- one draw from
 * softmax(outputs * inv_temp) per row and value of `random`; the key's value is that score.  The noise is this
 * library's own counter generator (berth draws from curand's Philox stream inside the fork's kernel, which is not part
 * of berth's tree): same distribution, different stream.  The logarithm is evaluated from exact steps in a fixed order,
 * so the CPU checker reproduces every key bit for bit from the stored outputs. */
int berth_exl3_linear_sample(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                             unsigned long long* best, int size_m, int size_k, int size_n, int k_bits, int codebook,
                             int out_fp32, float inv_temp, unsigned int random, int mode, void* stream);

/* The decode linear (size_m <= 32) with the residual stream added in its last step: c = residual + linear(a), fp32
 * [size_m][size_n]; c may be the residual itself (x += mlp(h2) in place).  Bit for bit what berth_exl3_linear with
 * out_fp32 = 1 followed by berth_ops_add_f32(residual, c, c) gives (crates/berth-engine/src/model.rs:976-1022), in
 * the launches of the linear alone (always the decode kernel: from 17 rows of a large matrix, where berth_exl3_linear
 * runs the split-K tensor-core kernel, equal within the accumulation tolerance).  No counterpart in berth. */
int berth_exl3_linear_add(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                          const void* residual, int size_m, int size_k, int size_n, int k_bits, int codebook,
                          void* stream);

/* The down projection of an MLP with the activation taken on the fly (size_m <= 32, the decode kernels):
 * c = [residual +] linear(silu(gate) * up), gate and up fp16 [size_m][size_k].  The rotation of the linear reads gate
 * and up instead of an activation buffer and forms silu(gate) * up with every step rounded to fp16 and the clamp to
 * +-act_limit (0 = none) exactly as berth_ops_silu_mul does, so c and a_had are bit for bit what
 * berth_ops_silu_mul(gate, up, act) + berth_exl3_linear(act) [+ berth_ops_add_f32] give from the same kernel
 * (crates/berth-engine/src/mlp.rs:128-160; the decode block's x += mlp(h2), model.rs:976-1022), one launch and one
 * buffer less.  residual may be null; when set it is fp32 [size_m][size_n], needs out_fp32 = 1 and may be c itself.
 * No counterpart in berth. */
int berth_exl3_linear_silu(const void* gate, const void* up, const void* trellis, void* c, const void* suh, void* a_had,
                           const void* svh, const void* residual, float act_limit, int size_m, int size_k, int size_n,
                           int k_bits, int codebook, int out_fp32, void* stream);

/* A stack of n_matrices equally shaped MUL1 linears applied to the same size_m <= 8 rows in ONE decode launch:
 * trellis_stack int16 [n][size_k/16][size_n/16][16*k_bits], suh_stack fp16 [n][size_k], svh_stack fp16 [n][size_n];
 * outputs c [n][size_m][size_n] and a_had [n][size_m][size_k].  What berth does for the gate and up projections of
 * an MLP with two berth_exl3_linear calls (crates/berth-engine/src/mlp.rs:118-150); a host that stores the two
 * projections one behind the other saves a launch, a pipeline ramp and a finishing kernel.  No counterpart in berth.
 * Other codebooks or more rows fail closed ("no linked kernel"). */
int berth_exl3_linear_stack(const void* a, const void* trellis_stack, void* c, const void* suh_stack, void* a_had,
                            const void* svh_stack, int n_matrices, int size_m, int size_k, int size_n, int k_bits,
                            int codebook, int out_fp32, void* stream);

/* Up to four MUL1 linears of different widths (same size_k, k_bits) applied to the same size_m <= 8 rows in ONE decode
 * launch: the q, k and v projections of an attention block, which berth runs as one berth_ops_mgemm call over column
 * slices (crates/berth-kernels/src/ops.rs:257-262, crates/berth-engine/src/model.rs q/k/v of the attention layers).
 * The five pointer lists and size_n_list are HOST arrays of n_matrices entries (device pointers of each matrix's
 * trellis, output [size_m][size_n_i], suh, a_had [size_m][size_k] and svh): with the addresses known on the host the
 * library encodes one TMA view per matrix and rotates inside the kernel, which the device-resident lists of
 * berth_ops_mgemm do not allow.  Per matrix the result is what berth_exl3_linear gives for one row of a MUL1 matrix
 * (same kernel).  Other codebooks or more rows fail closed ("no linked kernel").  No counterpart in berth. */
int berth_exl3_linear_multi(const void* a, const void* const* trellis_list, void* const* c_list,
                            const void* const* suh_list, void* const* a_had_list, const void* const* svh_list,
                            const int* size_n_list, int n_matrices, int size_m, int size_k, int k_bits, int codebook,
                            int out_fp32, void* stream);

/* ------------------------------------------------------------------ prefill linear (m > 1)
 * Replaces berth_prefill_exl3_linear (crates/berth-kernels/src/prefill_lin.rs:37-52,
 * crates/berth-kernels/csrc/prefill_lin/linear.cu:232-381).  w_scratch (fp16,
 * size_k*min(size_n,32768)) is required when size_m > 144, as in berth, but is not written:
 * the weight tiles are decoded straight into shared memory. */
int berth_prefill_exl3_linear(const void* a, const void* trellis, void* c, const void* suh,
                              void* a_had, const void* svh, void* w_scratch, int size_m,
                              int size_k, int size_n, int k_bits, int codebook, int c_fp32,
                              void* stream);
const char* berth_prefill_last_error(void);
const char* berth_prefill_last_launch(void);
/* Shape heuristic of crates/berth-kernels/csrc/prefill_lin/gemv.cu:72-101 (pure integer logic,
 * no CUDA call).  Kept for ABI parity; this library does not consult it. */
int berth_exl3_gemv_cfg(int cc, int size_m, int size_k, int size_n, int k_bits, int cb, int mode,
                        int narrow_coresident);

/* The two stages berth's prefill path is built from, exported so the decoded weight tiles
 * can be checked bit for bit (crates/berth-kernels/csrc/prefill_lin/api.h:70-84,
 * csrc/prefill_lin/reconstruct.cu:31-95).  Errors are reported through berth_prefill_last_error.
 *   reconstruct: unpacked fp16 [size_k][slice_n] <- columns [n_offset, n_offset+slice_n) of the
 *                trellis of a [size_k][full_n] matrix;
 *   had_r_128:   128-wide Hadamard / sqrt(128) on every 128-column block of every row, the fp16
 *                sign-scale vector applied before (pre_scale != 0) or after the transform;
 *                fp32 != 0 selects fp32 tensors, else fp16; output may alias input. */
int berth_prefill_reconstruct(void* unpacked, const void* packed, int size_k, int slice_n,
                              int full_n, int n_offset, int k_bits, int codebook, void* stream);
int berth_prefill_had_r_128(const void* input, void* output, const void* scale, int pre_scale,
                            int rows, int cols, int fp32, void* stream);

/* ------------------------------------------------------------------ ops
 * silu(gate)*up in fp16, every step rounded to fp16; out may alias gate or up
 * (crates/berth-kernels/src/ops.rs:82-89,507-520, csrc/ops/act.cu:35-69). */
int berth_ops_silu_mul(const void* gate, const void* up, void* out, int64_t numel,
                       float act_limit, void* stream);
/* c = a + b, fp32; c may alias a (crates/berth-kernels/src/ops.rs:91-97, csrc/ops/add.cu:29-54). */
int berth_ops_add_f32(const void* a, const void* b, void* c, int n, void* stream);
/* RMSNorm of the decode blocks: replaces berth_ops_rms_norm, berth_ops_rms_norm_f16 and berth_ops_rms_norm_res_in
 * (crates/berth-kernels/src/ops.rs:55-80,108-118, csrc/ops/norm.cu:129-224; call sites
 * crates/berth-engine/src/model.rs:793,854).  y fp16 [rows][dim] = ((v * r) * (weight + constant_bias)) * constant_scale,
 * r = 1 / sqrt(mean(v^2) + epsilon); v = x (fp32; fp16 for _f16), or for _res_in the fp32 residual row after
 * residual += x, written back in place.  weight: bfloat16 (weight_bf16 = 1; always for _f16) or fp16 [dim].
 * dim must be a multiple of 4.  Errors through berth_ops_last_error with berth's wording. */
int berth_ops_rms_norm(const void* x, const void* weight, void* y, int rows, int dim, float epsilon,
                       float constant_bias, float constant_scale, int weight_bf16, void* stream);
int berth_ops_rms_norm_f16(const void* x, const void* weight, void* y, int rows, int dim, float epsilon,
                           float constant_bias, float constant_scale, void* stream);
int berth_ops_rms_norm_res_in(const void* x, const void* weight, void* y, void* residual, int rows, int dim,
                              float epsilon, float constant_bias, float constant_scale, int weight_bf16,
                              void* stream);
const char* berth_ops_last_error(void);
const char* berth_ops_last_launch(void);

/* Plain fp16 GEMM c[m][n] = a[m][k] . b[k][n], row stride of c = ldc elements, fp32 accumulation
 * (crates/berth-kernels/src/prefill_lin.rs:54-64,163-205, csrc/prefill_lin/hgemm.cu:192-268).  As in berth
 * the work is cublasGemmEx; cuBLAS is loaded at the first call (dlopen of libcublas.so.12), the rest of
 * the library does not depend on it.  The prefill linear above does not use it: it never
 * materialises the fp16 weight. */
int berth_prefill_hgemm(const void* a, const void* b, void* c, int size_m, int size_k, int size_n,
                        int ldc, int c_fp32, void* stream);

/* Several trellis linears that share one input in one decode launch, sliced mode
 * (crates/berth-kernels/src/ops.rs:17-38,247-367, csrc/ops/mgemm.cu:125-334): slice i is a run of size_n
 * columns of a matrix of n_stride_list[i] columns; b_list[i] = address of the slice's first tile
 * (trellis + (n0 / 16) * 16 * k_bits * 2 bytes), svh_list[i] = svh + n0, c_ptrs[i] = out + n0 (row stride
 * n_stride_list[i] elements), had_src_list[i] = which matrix it was cut from; suh_list[s] = suh of
 * matrix s; a_had = num_had_src slabs of size_m * size_k fp16.  b_list, suh_list, svh_list, c_ptrs are
 * DEVICE arrays of device addresses, size_n_list / n_stride_list / had_src_list DEVICE int arrays with
 * one entry per slice (bszm_out of them); bszm_in = 1.  c carries only the output type.  Returns a
 * positive tag (1, 2 or 4: the launch's token groups) or -1.  Differences from berth: every K and
 * codebook is linked, size_m up to 32, no autotune; size_k must be a multiple of 128 and size_n of 256
 * (128 above 4 bits).  Uniform mode (size_n_list, c_ptrs, n_stride_list and had_src_list all NULL, num_had_src = 0;
 * crates/berth-kernels/csrc/ops/mgemm.cu:164-198): bszm_out equally shaped matrices (b_list, suh_list, svh_list with
 * bszm_out entries), outputs c (bszm_out, size_m, size_n), inputs a (bszm_in, size_m, size_k) with bszm_in = 1 (one
 * input for all) or bszm_out (one each), a_had bszm_out slabs; at most 2048 matrices. */
int berth_ops_mgemm(const void* a, const void* b_list, void* c, const void* suh_list, void* a_had,
                    const void* svh_list, int size_m, int size_k, int size_n, int k_bits,
                    int codebook, int c_fp32, int bszm_in, int bszm_out, const int* size_n_list,
                    const void* c_ptrs, const int* n_stride_list, const int* had_src_list,
                    int num_had_src, void* stream);
/* Key of berth's multi-linear autotune cache (csrc/ops/mgemm.cu:61-91,277-294), kept for tooling that
 * reads that cache; nothing here autotunes. */
uint64_t berth_ops_mgemm_tune_key(int size_m, int size_k, int size_n, int k_bits, int c_fp32,
                                  int device, int cc, int sms, int cb, int bszm_in, int bszm_out,
                                  int sliced);

/* ------------------------------------------------------------------ MoE layer
 * berth has the shape contract of the A3B mixture-of-experts block (crates/berth-plan/src/plan.rs:43-57,
 * 204-219; crates/berth-plan/src/shape.rs:59-69) but no operator for it
 * (crates/berth-engine/src/model.rs:404-411), so these entry points have no counterpart in
 * berth's FFI; they follow the same conventions. */
typedef struct berth_moe_weights {
    int hidden, inter, shared_inter, n_experts, top_k, k_bits, codebook;
    const void* w_router;        /* fp16 [hidden][n_experts] */
    const float* router_bias;    /* fp32 [n_experts] or NULL */
    /* expert stacks: trellis (E, K/16, N/16, 16*k_bits), suh [E][K], svh [E][N].
     * Two optional placements save launches without changing a bit of the result: a shared expert of the experts'
     * shape stored directly behind every stack (as matrix E) runs inside the grouped expert launches; the up stack
     * (trellis and svh, shared expert included) stored directly behind the gate stack lets gate and up run as one
     * grouped launch.  The library recognises both from the pointers. */
    const void *gate_trellis, *up_trellis, *down_trellis;
    const void *gate_suh, *gate_svh, *up_suh, *up_svh, *down_suh, *down_svh;
    /* shared expert (shared_inter > 0) */
    const void *sh_gate_trellis, *sh_up_trellis, *sh_down_trellis;
    const void *sh_gate_suh, *sh_gate_svh, *sh_up_suh, *sh_up_svh, *sh_down_suh, *sh_down_svh;
} berth_moe_weights;

/* Router: logits = x . w_router (+ bias) in fp32 with a fixed summation order (32 chunk sums of
 * hidden/32 sequential fmaf, then an xor tree), top-k with ties to the lower expert index,
 * weights = softmax over the selected logits.
 * x fp16 [T][hidden]; topk_idx int32 [T][k]; topk_w fp32 [T][k]; logits fp32 [T][E] scratch/output. */
int berth_moe_router_topk(const void* x, const void* w_router, const float* router_bias,
                          int32_t* topk_idx, float* topk_w, float* logits, int T, int hidden,
                          int n_experts, int top_k, void* stream);
/* Bytes of caller-provided scratch berth_moe_layer needs for T tokens (the library allocates
 * nothing per layer). */
size_t berth_moe_workspace_bytes(int T, int hidden, int inter, int shared_inter, int n_experts,
                                 int top_k);
/* The whole layer on one GPU: router, dispatch, grouped gate/up/SiLU/down over the routed rows,
 * shared expert, weighted combine.  x fp16 [T][hidden]; out fp32 [T][hidden]; topk_idx / topk_w
 * receive the routing ([T][k]).  Expert outputs are rounded to fp16 and combined in fp32 in slot
 * order, shared expert last. */
int berth_moe_layer(const berth_moe_weights* w, const void* x, int T, void* out, int32_t* topk_idx,
                    float* topk_w, void* workspace, size_t workspace_bytes, void* stream);
/* The stages of the layer one by one, for hosts that put a collective between them (expert
 * parallelism).  `ews` is caller-provided scratch of berth_moe_experts_workspace_bytes(max_rows,
 * n_local, hidden, inter, max_rows_per_expert) bytes; the same five values must be passed to
 * berth_moe_sort_rows and berth_moe_experts, which share the problem table inside it.
 *   sort_rows: stable sort of n entries by key (expert id) restricted to [e0, e0 + n_local):
 *              perm[pos] = entry, inv[entry] = pos, offsets_out[0..n_local] = first row of each
 *              expert (optional), and the problem table of the following berth_moe_experts call;
 *   gather:    dst[i][:] = src[index[i] / div][:], fp16 rows of `hidden` elements;
 *   experts:   yr = down(silu(gate(xr)) * up(xr)) row by row, xr fp16 [n_rows][hidden] sorted by
 *              expert as sort_rows left them; w holds the LOCAL expert stacks (n_experts = n_local);
 *   combine:   out[t] = sum_s topk_w[t][s] * y[inv[t*k+s]] (+ ysh[t]), fp32. */
size_t berth_moe_experts_workspace_bytes(int max_rows, int n_local, int hidden, int inter,
                                         int max_rows_per_expert);
int berth_moe_sort_rows(const int32_t* keys, int n, int e0, int n_local, int32_t* perm, int32_t* inv,
                        int32_t* offsets_out, void* ews, size_t ews_bytes, int max_rows, int hidden,
                        int inter, int max_rows_per_expert, void* stream);
int berth_moe_gather(const void* src, const int32_t* index, int div, int n, void* dst, int hidden,
                     void* stream);
int berth_moe_experts(const berth_moe_weights* w, const void* xr, void* yr, int n_rows, void* ews,
                      size_t ews_bytes, int max_rows, int max_rows_per_expert, void* stream);
int berth_moe_combine(const void* y, const int32_t* inv, const float* topk_w, const void* ysh,
                      void* out, int T, int hidden, int top_k, void* stream);
/* The two compute sides of an expert-parallel layer as one call each (the host puts its all-to-alls
 * between them; no counterpart in berth).
 *   ep_send:    route the T local tokens over all n_experts, sort the (token, slot) pairs by expert
 *               (= by destination rank, experts being split in contiguous blocks) and gather their
 *               rows.  Out: topk_idx/topk_w [T][k]; inv[T*k] = position of pair (t, s) in the sorted
 *               order; send_rows fp16 [T*k][hidden] in that order; counts[n_experts] rows per expert.
 *   ep_experts: recv_rows fp16 [n_rows][hidden] = the rows of source 0, 1, .. world-1, each source's
 *               rows sorted by local expert, cnt_recv[world][n_local] of them per (source, expert).
 *               Regroups by local expert, runs the experts (w holds the LOCAL stacks) and writes the
 *               outputs in arrival order to back [n_rows][hidden].  With ysh != NULL the shared expert,
 *               which must then be stored behind the stacks as matrix n_local, runs in the same
 *               launches on x_local [T_local][hidden] -> ysh [T_local][hidden].  rows_hint = the rows
 *               per expert to size the problems for (see berth_moe_experts). */
size_t berth_moe_ep_send_workspace_bytes(int T, int n_experts, int top_k);
int berth_moe_ep_send(const void* x, int T, const void* w_router, const float* router_bias, int hidden,
                      int n_experts, int top_k, int32_t* topk_idx, float* topk_w, int32_t* inv,
                      void* send_rows, int32_t* counts, void* ws, size_t ws_bytes, void* stream);
size_t berth_moe_ep_experts_workspace_bytes(int max_rows, int max_tokens, int world, int n_local,
                                            int hidden, int inter);
int berth_moe_ep_experts(const berth_moe_weights* w, const void* recv_rows, int n_rows,
                         const int32_t* cnt_recv, int world, const void* x_local, int T_local, void* back,
                         void* ysh, void* ws, size_t ws_bytes, int max_rows, int max_tokens, int rows_hint,
                         void* stream);
/* The same two sides with the exchange done by the kernels themselves, over peer memory (the ranks of
 * one NVSwitch box; no collective library call, no host synchronisation; no counterpart in berth).
 * The host allocates four symmetric buffers on every rank and passes the per-rank device addresses
 * (host arrays of `world` pointers, world <= 8):
 *   cnt_all    int32 [world][n_experts]      rows per expert of every rank (each rank writes its row everywhere)
 *   flags      uint32 [3][8], zero at start  flag barriers: counts published / rows delivered / outputs returned
 *   recv_rows  fp16 [max_rows][hidden]       routed rows, written by their sources at their final, expert-sorted place
 *   ret_rows   fp16 [max_send][hidden]       expert outputs, written by the experts' ranks at the row's send position
 * `epoch` must grow by one with every layer call, the same on all ranks.  A rank calls p2p_send (route,
 * sort, publish counts, deliver rows), then p2p_experts (experts on what arrived, plus the shared expert
 * of its own T_local tokens when ysh != NULL -- it must then sit behind the stacks as matrix n_local --,
 * return the outputs), then berth_moe_combine on its own ret_rows with the inv / topk_w of p2p_send.
 * max_rows bounds the rows a rank can receive plus its own T_local; a row that would not fit is dropped
 * and reported in berth_device_status (bit 64); a peer that never arrives ends the wait after about half
 * a second (bit 32). */
size_t berth_moe_p2p_send_workspace_bytes(int T, int n_experts, int top_k, int world);
int berth_moe_p2p_send(const void* x, int T, const void* w_router, const float* router_bias, int hidden,
                       int n_experts, int top_k, int32_t* topk_idx, float* topk_w, int32_t* inv, int rank,
                       int world, unsigned epoch, const void* const* cnt_all, const void* const* flags,
                       const void* const* recv_rows, int max_rows, void* ws, size_t ws_bytes, void* stream);
size_t berth_moe_p2p_experts_workspace_bytes(int max_rows, int n_local, int hidden, int inter);
int berth_moe_p2p_experts(const berth_moe_weights* w, const void* x_local, int T_local, void* ysh, int rank,
                          int world, unsigned epoch, int n_experts_total, int top_k, int send_tokens,
                          const void* const* cnt_all, const void* const* flags, const void* const* recv_rows,
                          const void* const* ret_rows, int max_rows, int max_send, int rows_hint, void* send_ws,
                          void* ws, size_t ws_bytes, void* stream);
const char* berth_moe_last_error(void);
const char* berth_moe_last_launch(void);

#ifdef __cplusplus
}
#endif
#endif /* BERTH_B200_H */
