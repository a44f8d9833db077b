/* C ABI of gllm_b200. Thread-safe: every call takes the interpreter lock of the embedded Python runtime.
 *
 * The first five entry points are call-compatible with the reference's C ABI (src/ffi.rs:44,70,82,133,152):
 *   gllm_init(model_id, kind)                 kind: 0 chat, 1 embedding, 2 reranker, 3 classifier
 *   gllm_destroy(ctx)
 *   gllm_generate(ctx, prompt, max_tokens, temperature, top_k, top_p, thinking_budget)
 *                                             returns {text, error} BY VALUE; exactly one of the two is non-NULL
 *                                             thinking_budget: 0 disabled, negative unlimited, positive max tokens
 *   gllm_free_generate_result(&result)        frees the two strings and NULLs them
 *   gllm_client_version()
 * so a client built against the reference links and runs unchanged. Device, dtype and engine limits of a context made
 * by gllm_init come from the environment variable GLLM_FFI_OPTIONS (a JSON object, see gllm_init_with_options).
 *
 * The *_ex / *_with_options entry points and gllm_embed / gllm_rerank_score are additions: a richer result (token ids,
 * finish reason), explicit options, and the embedding / reranking models that `kind` selects, reachable from C.
 */
#ifndef GLLM_FFI_H
#define GLLM_FFI_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef struct GllmContext GllmContext;

typedef struct {
  char* text;  /* generated text (UTF-8, NUL terminated) or NULL on failure */
  char* error; /* NULL on success, else the error message */
} GllmGenerateResult;

GllmContext* gllm_init(const char* model_id, uint32_t kind);
void gllm_destroy(GllmContext* ctx);
GllmGenerateResult gllm_generate(GllmContext* ctx, const char* prompt, uint32_t max_tokens, float temperature,
                                 uint32_t top_k, float top_p, int32_t thinking_budget);
void gllm_free_generate_result(GllmGenerateResult* result);
const char* gllm_client_version(void);

/* ---- additions ---- */
typedef struct {
  char* text;            /* UTF-8, NUL terminated; owned by the result */
  int* token_ids;
  int num_tokens;
  int prompt_tokens;
  int finish_reason;     /* 1 eos, 2 length, 3 aborted, 4 veto */
  int error;             /* 0 = ok */
  char* error_message;
} GllmGenerateResultEx;

/* model_id: a preset name ("tiny-llama", "qwen3-8b", ...) for random-init weights, or a path / hub id.
 * options_json: optional JSON object: {"device": "cuda:0"|"cpu", "dtype": "bf16"|"fp32", "max_num_seqs": n, ...}.
 * Returns NULL on failure; gllm_last_init_error() says why. */
GllmContext* gllm_init_with_options(const char* model_id, uint32_t kind, const char* options_json);
GllmGenerateResultEx* gllm_generate_ex(GllmContext* ctx, const char* prompt, uint32_t max_tokens, float temperature,
                                       uint32_t top_k, float top_p, int32_t thinking_budget);
void gllm_free_generate_result_ex(GllmGenerateResultEx* r);
const char* gllm_last_init_error(void);
/* Embedding of `text` (L2-normalised) into out[0..capacity); returns the embedding dimension, or -1 on failure. */
int gllm_embed(GllmContext* ctx, const char* text, float* out, int capacity);
/* Relevance score of `document` for `query`; returns 0 on success. */
int gllm_rerank_score(GllmContext* ctx, const char* query, const char* document, float* score);

#ifdef __cplusplus
}
#endif
#endif
