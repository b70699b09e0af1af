/* EXL3 checkpoint reader of libberth_b200.so: the load-time half of the quantized linear path.
 *
 * Replaces, behind a C ABI, what berth's `berth-exl3` crate gives its engine:
 *   Checkpoint::open / linears / other_tensors   crates/berth-exl3/src/checkpoint.rs:30-72
 *   TensorInfo, TensorIndex                       crates/berth-exl3/src/safetensors.rs:14-66
 *   LinearExl3, Bitrate, Codebook, HadamardScale  crates/berth-exl3/src/linear.rs:14-138
 *   LinearExl3::unpack_{input,output}_signs       crates/berth-exl3/src/linear.rs:140-155
 *   unpack_signs                                  crates/berth-exl3/src/signs.rs:25-45
 * Host memory only; nothing here touches a GPU.  Every function that can fail returns 0 on success and -1 on
 * error with the message in berth_ckpt_last_error() (thread-local, valid until the next call on the thread).
 * Messages name the offending tensor or field first, as berth's Error::BadField does.  berth_config_* reads config.json
 * (ModelConfig / QuantizationConfig of crates/berth-exl3/src/config.rs). */
#ifndef BERTH_B200_CHECKPOINT_H
#define BERTH_B200_CHECKPOINT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct berth_ckpt berth_ckpt;

/* safetensors dtypes, in the order of crates/berth-exl3/src/dtype.rs:6-23 */
enum {
    BERTH_DT_BOOL = 0, BERTH_DT_U8, BERTH_DT_I8, BERTH_DT_I16, BERTH_DT_U16, BERTH_DT_I32, BERTH_DT_U32, BERTH_DT_I64,
    BERTH_DT_U64, BERTH_DT_F16, BERTH_DT_BF16, BERTH_DT_F32, BERTH_DT_F64, BERTH_DT_F8_E4M3, BERTH_DT_F8_E5M2, BERTH_DT_F8_E8M0
};

/* One tensor of the index.  Strings stay valid until berth_ckpt_close. */
typedef struct {
    const char* name;
    const char* shard;      /* path of the file that holds it */
    int dtype;              /* BERTH_DT_* */
    int rank;               /* at most 8 */
    uint64_t shape[8];
    uint64_t offset;        /* absolute byte offset in the shard */
    uint64_t length;        /* bytes */
} berth_tensor_info;

/* One EXL3 linear, grouped by the prefix of its `.trellis` tensor. */
typedef struct {
    const char* prefix;
    berth_tensor_info trellis;        /* I16, rank 3: [K/16][N/16][16 * bits] */
    berth_tensor_info input_scale;    /* `suh` (F16) if present, else packed `su` (I16) */
    berth_tensor_info output_scale;   /* `svh` (F16) if present, else packed `sv` (I16) */
    berth_tensor_info bias;           /* valid if has_bias */
    int input_packed, output_packed, has_bias;
    int codebook;                     /* the kernels' numbering: 0 = default (3INST), 1 = mcg, 2 = mul1 */
    int bits_x2;                      /* bits per weight times two: 8 = 4 bpw, 5 = 2.5 bpw (half rates need mul1) */
} berth_linear_info;

/* Opens a checkpoint directory: model.safetensors.index.json (weight_map, optional metadata.total_size, which is
 * checked against the tensor bytes) or a single model.safetensors. */
int berth_ckpt_open(const char* directory, berth_ckpt** out);
void berth_ckpt_close(berth_ckpt* ckpt);

int64_t berth_ckpt_n_tensors(const berth_ckpt* ckpt);
int64_t berth_ckpt_n_linears(const berth_ckpt* ckpt);   /* sorted by prefix */
int64_t berth_ckpt_n_others(const berth_ckpt* ckpt);    /* tensors that belong to no linear, in name order */
int berth_ckpt_tensor_at(const berth_ckpt* ckpt, int64_t i, berth_tensor_info* out);   /* name order */
int berth_ckpt_tensor(const berth_ckpt* ckpt, const char* name, berth_tensor_info* out);
int berth_ckpt_linear_at(const berth_ckpt* ckpt, int64_t i, berth_linear_info* out);
int berth_ckpt_linear(const berth_ckpt* ckpt, const char* prefix, berth_linear_info* out);
int berth_ckpt_other_at(const berth_ckpt* ckpt, int64_t i, berth_tensor_info* out);

/* Copies the tensor's bytes into dst (host memory); dst_bytes must equal the tensor's length. */
int berth_ckpt_read(const berth_ckpt* ckpt, const char* name, void* dst, uint64_t dst_bytes);
/* The linear's input (output_side = 0) or output scale as fp16 bit patterns: a copy of `suh` / `svh`, or the
 * packed signs unpacked to +-1.0.  dst_halves must equal the channel count. */
int berth_ckpt_scale_f16(const berth_ckpt* ckpt, const char* prefix, int output_side, uint16_t* dst, uint64_t dst_halves);

/* Packed little-endian int16 sign words -> fp16 bit patterns: bit i of a word is element i, a set bit is -1.0
 * (0xBC00), a clear bit +1.0 (0x3C00).  `bytes` must be even; out receives bytes * 8 values. */
int berth_unpack_signs(const void* packed_le, uint64_t bytes, uint16_t* out);

/* config.json: the text stack and the quantization block (crates/berth-exl3/src/config.rs:52-160).  Text fields are read
 * from `text_config` when that object holds the key, else from the top level; `architectures` and `quantization_config`
 * are top-level; unknown keys are ignored; integers may be written as integer-valued floats.  Optional integers are -1
 * and optional strings NULL when absent.  Errors through berth_ckpt_last_error with berth's wording: "missing field `x`"
 * or "field `x`: detail".  Strings and the layer_types array stay valid until berth_config_free. */
typedef struct berth_config_strings berth_config_strings;
typedef struct {
    const char* arch_string;                 /* architectures[0] */
    uint32_t num_hidden_layers, hidden_size, head_dim, num_attention_heads, num_key_value_heads, vocab_size;
    int tie_word_embeddings, attn_output_gate;
    uint32_t linear_conv_kernel_dim, linear_num_key_heads, linear_num_value_heads, linear_key_head_dim, linear_value_head_dim;
    int64_t intermediate_size, num_experts, num_experts_per_tok, moe_intermediate_size, shared_expert_intermediate_size;
    int64_t n_layer_types;                   /* = num_hidden_layers */
    const char* const* layer_types;          /* "linear_attention", "full_attention", or any other string as written */
    /* quantization_config */
    const char* quant_method;
    double bits;
    uint32_t head_bits;
    const char* codebook;
    const char* version;
    const char* out_scales;
    int64_t vision_bits, mtp_bits, calibration_rows, calibration_cols;
    berth_config_strings* strings;           /* owner of the strings above */
} berth_model_config;
int berth_config_parse(const char* json, uint64_t bytes, berth_model_config** out);
int berth_config_open(const char* directory, berth_model_config** out);   /* <directory>/config.json */
void berth_config_free(berth_model_config* config);

const char* berth_ckpt_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
