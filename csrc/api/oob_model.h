/* C ABI of the decode-path kernels used by the tensor-parallel model runner: rotary embedding fused with the
 * KV-cache write, SwiGLU activation, and grouped-query decode attention over a static cache.
 *
 * Capability parity: the reference serves models through vLLM and leaves these ops to it
 * (patches/vllm/v0.25.0/vllm/model_executor/models/qwen2.py); the model runner of this library needs them so
 * that a decode step is a short, fixed sequence of kernels that one CUDA graph replays.
 *
 * All functions return 0 or a negative oob_status_t (see oob.h); matrices are 16-bit (OOB_F16 / OOB_BF16).
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

typedef struct {
  int dtype;
  int B, T;          /* sequences and tokens per sequence in qkv ([B*T, (H + 2*KV) * hd], row-major) */
  int H, KV, hd;     /* local query heads, local KV heads, head size (multiple of 8; rotation pairs are (2i, 2i+1)) */
  const void* qkv;
  void* q_out;       /* [B*T, H * hd] */
  void* k_cache;     /* this layer's cache: [batch][KV][max_len][hd] */
  void* v_cache;
  int64_t cache_batch_stride; /* elements between sequences of the cache */
  int max_len;
  int batch0;        /* first cache slot of this call's sequences */
  const float* cos_table; /* [max_len, hd/2] fp32 */
  const float* sin_table;
  const int64_t* pos_dev; /* device scalar: position of token 0 of every sequence; NULL = pos0 */
  int pos0;
} oob_rope_args_t;
int oob_rope_kv_write(const oob_rope_args_t* a, void* stream);

/* out[r, j] = silu(gu[r, j]) * gu[r, F + j]; gu is [rows, 2F] with leading dimension ld_gu, out is [rows, F]
 * contiguous; F a multiple of 8. */
int oob_silu_mul(int dtype, const void* gu, int64_t ld_gu, void* out, int rows, int F, void* stream);

typedef struct {
  int dtype;
  int B, H, KV;       /* sequences, local query heads, local KV heads (H / KV <= 16); head size is 128 */
  const void* q;      /* [B, H, 128] */
  const void* k_cache;/* this layer's cache: [batch][KV][max_len][128] */
  const void* v_cache;
  int64_t cache_batch_stride;
  int max_len;
  int batch0;
  void* out;          /* [B, H * 128] */
  const int64_t* pos_dev; /* device scalar: index of the newest key; context length = *pos_dev + 1.  NULL = len */
  int len;
  float scale;        /* softmax scale (1/sqrt(128) for standard attention) */
  int splits;         /* CTAs per (sequence, KV head) along the keys; 0 = choose from B * KV and len_bound */
  int len_bound;      /* upper bound of the context length for this launch (sizes the key chunks); 0 = max_len */
  float* workspace;   /* fp32, oob_attn_decode_workspace_bytes(B, H, splits) bytes; may be NULL when splits == 1 */
} oob_attn_decode_args_t;
int oob_attn_decode(const oob_attn_decode_args_t* a, void* stream);
/* Split count oob_attn_decode picks for splits == 0. */
int oob_attn_decode_auto_splits(int B, int KV, int len_bound);
uint64_t oob_attn_decode_workspace_bytes(int B, int H, int splits);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
