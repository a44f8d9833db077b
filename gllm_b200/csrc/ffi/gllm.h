/* C ABI of gllm_b200. Thread-safe: every call takes the interpreter lock of the embedded Python runtime.
 *
 * Reference parity: gllm_init / gllm_destroy / gllm_generate / gllm_free_generate_result / gllm_client_version
 * (src/ffi.rs:44,70,82,133,152).
 */
#ifndef GLLM_FFI_H
#define GLLM_FFI_H
#ifdef __cplusplus
extern "C" {
#endif

typedef struct gllm_client gllm_client;

typedef struct {
  char* text;            /* UTF-8, NUL terminated; owned by the result */
  int* token_ids;
  int num_tokens;
  int prompt_tokens;
  int finish_reason;     /* 1 eos, 2 length, 3 aborted, 4 veto */
  int error;             /* 0 = ok */
  char* error_message;
} gllm_generate_result;

/* model_id: a preset name ("tiny-llama", "qwen3-8b", ...) for random-init weights, or a path / hub id.
 * options_json: optional JSON object: {"device": "cuda:0"|"cpu", "dtype": "bf16"|"fp32", "max_num_seqs": n, ...}.
 * Returns NULL on failure; gllm_last_init_error() says why. */
gllm_client* gllm_init(const char* model_id, const char* options_json);
void gllm_destroy(gllm_client* c);
gllm_generate_result* gllm_generate(gllm_client* c, const char* prompt, int max_tokens, float temperature, int top_k,
                                    float top_p);
void gllm_free_generate_result(gllm_generate_result* r);
const char* gllm_client_version(void);
const char* gllm_last_init_error(void);

#ifdef __cplusplus
}
#endif
#endif
