/*
 * CPU oracle for the EXL3 trellis-linear / A3B-MoE path.  TEST INFRASTRUCTURE ONLY:
 * nothing that ships (the CUDA library, the Python host package) may link, import or
 * call this file; it exists so tests and the benchmark's cpu_baseline leg have a
 * checker that shares no code with the CUDA kernels.
 *
 * PARITY UNPINNED for the trellis / codebook / Hadamard arithmetic.  berth links that
 * arithmetic from an external exllamav3 fork (git tree de35ffbe336bdc6d617e49e208cd7c730a789787,
 * crates/berth-kernels/build.rs:16) that is not vendored, and its golden outputs
 * (testdata/exl3_ref) need a 27B checkpoint that is not available.  This file restates
 * the published algorithm (QTIP bitshift trellis + computed codebooks, Tseng et al. 2024,
 * arXiv:2406.11235; EXL3 format notes of exllamav3) and honours every fact berth's own
 * sources state about the format; the remaining free choices are fixed in the
 * comment at the top of exl3_oracle.c ("spec v0").  The pieces that berth's tree does pin are pinned:
 * silu_mul against testdata/kernels/ops/silu.*.bin (bit-exact), add_f32 against
 * add.*.bin, unpack_signs against the known answers of crates/berth-exl3/src/signs.rs:52-91,
 * exl3_gemv_cfg against crates/berth-kernels/src/prefill_lin.rs:386-442 and the GEMM
 * tune key against crates/berth-kernels/src/lib.rs:224-233.
 */
#ifndef EXL3_ORACLE_H
#define EXL3_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- fp16 <-> fp32/fp64, round to nearest even, bit patterns in uint16_t ---- */
float    exl3o_h2f(uint16_t h);
uint16_t exl3o_f2h(float f);
uint16_t exl3o_d2h(double d);

/* ---- format: crates/berth-exl3/src/signs.rs:25-45 ---- */
/* n_words packed int16 sign words -> 16*n_words fp16 bit patterns (0x3C00 / 0xBC00). */
void exl3o_unpack_signs(const uint16_t* packed, int64_t n_words, uint16_t* out);

/* ---- codebook: one 16-bit trellis state -> one fp16 weight (bit pattern) ----
 * cb 0 = 3INST, 1 = MCG, 2 = MUL1 (selector values of crates/berth-kernels/src/lib.rs:49-63). */
uint16_t exl3o_codebook(uint32_t state, int cb);

/* ---- tile: 16*bits uint16 words -> 256 states / 16x16 fp16 weights ----
 * states[t], t = 0..255 in trellis order; tile[row*16 + col] in matrix order. */
void exl3o_tile_states(const uint16_t* words, int bits, uint16_t* states);
void exl3o_tile_coords(int t, int* row, int* col);
void exl3o_decode_tile(const uint16_t* words, int bits, int cb, uint16_t* tile);

/* ---- whole matrix: trellis (K/16, N/16, 16*bits) -> fp16 W[K][ldw], columns
 * [n_offset, n_offset + slice_n) of a matrix whose full width is full_n
 * (crates/berth-kernels/csrc/prefill_lin/reconstruct.cu:69-95). */
void exl3o_reconstruct(const uint16_t* trellis, int size_k, int full_n, int n_offset,
                       int slice_n, int bits, int cb, uint16_t* w, int ldw);

/* ---- 128-wide Hadamard over each contiguous 128-column block of each row, times
 * 1/sqrt(128) (0.088388347648f), with the sign-scale vector applied before (pre_scale=1)
 * or after (pre_scale=0) the transform (crates/berth-kernels/csrc/prefill_lin/reconstruct.cu:31-67).
 * fp32 = 0: fp16 in/out; fp32 = 1: fp32 in/out.  scale is fp16[cols] or NULL. */
void exl3o_had_r_128(const void* in, void* out, const uint16_t* scale, int pre_scale,
                     int rows, int cols, int fp32);

/* ---- the linear: y = H(H(x*suh)/s . W)/s * svh  (csrc/prefill_lin/linear.cu:201-230) ----
 * a fp16[m][k]; a_had fp16[m][k] out (may be NULL); c fp16 or fp32 [m][n].
 * fp32 accumulation in ascending k.  Returns 0, or -1 on a bad shape. */
int exl3o_linear(const uint16_t* a, const uint16_t* trellis, void* c, const uint16_t* suh,
                 uint16_t* a_had, const uint16_t* svh, int size_m, int size_k, int size_n,
                 int bits, int cb, int out_fp32);
/* Same product evaluated in fp64 from the fp16 inputs and the fp16 decoded weights,
 * with no intermediate rounding: the yardstick for the 1e-2 / 1e-3 tolerances. */
int exl3o_linear_f64(const uint16_t* a, const uint16_t* trellis, double* c, const uint16_t* suh,
                     const uint16_t* svh, int size_m, int size_k, int size_n, int bits, int cb);

/* ---- silu(gate) * up, fp16, every step rounded to fp16
 * (crates/berth-kernels/csrc/ops/act.cu:35-69; pinned by testdata/kernels/ops/silu.*.bin) */
uint16_t exl3o_hexp_neg(uint16_t g);   /* fp16(exp(-g)); equals the correctly rounded value at all but 2 of the 65536 inputs */
void exl3o_sample_keys(const float* outputs, int rows, int n, float inv_temp, uint32_t random, int mode, uint64_t* keys,
                       float* scores);
void exl3o_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t numel,
                    float act_limit);
/* c = a + b in fp32 (crates/berth-kernels/csrc/ops/add.cu:23-27). */
void exl3o_add_f32(const float* a, const float* b, float* c, int64_t n);
/* RMSNorm (berth_ops_rms_norm / _f16 / _res_in); the summation order is stated at the definition. */
void exl3o_rms_norm(const void* x, int x_is_f16, const uint16_t* weight, int weight_bf16, uint16_t* y, float* residual,
                    int rows, int dim, float epsilon, float constant_bias, float constant_scale);

/* ---- host-only integer logic of the boundary ---- */
/* crates/berth-kernels/csrc/prefill_lin/gemv.cu:72-101 */
int exl3o_gemv_cfg(int cc, int m, int k, int n, int bits, int cb, int mode, int narrow_coresident);
/* crates/berth-kernels/csrc/linear.cu:65-104,345-358 */
uint64_t exl3o_gemm_tune_key(int m, int k, int n, int bits, int out_fp32, int device, int cc,
                             int sms, int cb);

/* ---- MoE layer (no reference implementation exists in berth; the contract is the
 * benchmark configuration: softmax router, top-k with ties to the lower expert index,
 * weights renormalised over the selected experts, SiLU-gated experts, shared expert) ---- */
/* logits fp32[T][E]: 32 chunk sums of H/32 sequential fmaf each, then a fixed xor tree. */
void exl3o_router_logits(const uint16_t* x, const uint16_t* w_router, const float* bias,
                         float* logits, int T, int H, int E);
void exl3o_router_topk(const float* logits, int32_t* topk_idx, float* topk_w, int T, int E, int k);

typedef struct {
    int hidden, inter, shared_inter, n_experts, top_k, bits, cb;
    const uint16_t* w_router;              /* fp16 [hidden][n_experts] */
    const float* router_bias;              /* fp32 [n_experts] or NULL */
    const uint16_t *gate_trellis, *up_trellis, *down_trellis;   /* expert stacks */
    const uint16_t *gate_suh, *gate_svh, *up_suh, *up_svh, *down_suh, *down_svh;
    const uint16_t *sh_gate_trellis, *sh_up_trellis, *sh_down_trellis;  /* shared expert or NULL */
    const uint16_t *sh_gate_suh, *sh_gate_svh, *sh_up_suh, *sh_up_svh, *sh_down_suh, *sh_down_svh;
} exl3o_moe_weights;

/* out fp32[T][hidden]; topk_idx / topk_w may be NULL.  Expert outputs are rounded to fp16,
 * then combined in fp32 in slot order, shared expert last. */
int exl3o_moe_layer(const exl3o_moe_weights* w, const uint16_t* x, int T, float* out,
                    int32_t* topk_idx, float* topk_w);
/* Same layer with every linear and the combine in fp64 (routing taken from topk_idx). */
int exl3o_moe_layer_f64(const exl3o_moe_weights* w, const uint16_t* x, int T,
                        const int32_t* topk_idx, const float* topk_w, double* out);

int exl3o_num_threads(void);
void exl3o_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
