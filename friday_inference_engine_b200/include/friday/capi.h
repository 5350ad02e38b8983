/* The C interface of libfriday_engine: what the Python package, bin/friday and bin/trace_run are bindings over.
 *
 * Every function returns 0 on success and a non-zero error kind otherwise (the values of friday::ErrorKind plus
 * 100: 100 other, 101 configuration, 102 weights, 103 step, 104 cache, 105 cache full, 106 generation, 107 kernel,
 * 108 build); the message is read with friday_last_error(), and for a weights error friday_last_error_detail()
 * gives the lists (missing, unexpected, wrong_shape) as JSON.  Strings that functions hand back stay valid until
 * the same thread's next call into the library.  Handles are opaque pointers; a handle is freed by its _free. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FridayTensor {      /* same layout as friday::Tensor */
    void* data;
    int dtype;                     /* 0 float32, 1 bfloat16, 2 int32 */
    int ndim;
    int64_t shape[4];
    int64_t ld;
} FridayTensor;

typedef struct FridayKV {          /* keys and values of one cache entry as an attention kernel sees them */
    void* k_pool;
    void* v_pool;
    int pool_pages;
    const int* block_table;
    int table_width, page_size, window, n_kv_heads, head_dim, dtype, write;
} FridayKV;

typedef struct FridayGeometry {    /* the geometry of a step (friday::StepContext); per-sequence arrays may be null */
    int rows, n_seqs, max_q_len, max_kv_len, decode;
    const int* row_seq;
    const int* row_pos;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_pos0;
} FridayGeometry;

const char* friday_last_error(void);
const char* friday_last_error_detail(void);
int friday_set_builder(int (*build)(const char* family));
int friday_load_plugin(const char* path);
const char* friday_loaded_libraries(void);

/* configuration, registry, description of a model as data */
int friday_read_config(const char* config_json, const char** typed_json);
int friday_registered(const char* what, const char** json_list);      /* "architectures" or a part category */
int friday_describe_model(const char* config_json, const char** json);

/* weights */
int friday_write_random_model(const char* dir, const char* config_json, uint64_t seed, const char* dtype, int shards);
int friday_check_weights(const char* model_dir);
/* in which dtype every tensor of the folder would be kept by an engine of `dtype` (name, dtype, into) */
int friday_storage_plan(const char* model_dir, const char* dtype, const char** json);
int friday_random_tensor(uint64_t seed, const char* name, int one, int64_t count, float* out);
int friday_safetensors_open(const char* path_or_dir, void** handle);
int friday_safetensors_list(void* handle, const char** json);
int friday_safetensors_read(void* handle, const char* name, void* out, size_t bytes);
void friday_safetensors_free(void* handle);
int friday_safetensors_write(const char* path, const char* header_json, const void* const* blobs, const char* metadata_json);

/* the cache's book-keeping alone (no device memory) */
int friday_cache_new(const char* requests_json, int64_t max_tokens, int max_seq_tokens, int max_slots, void** handle);
void friday_cache_free(void* cache);
int friday_cache_alloc_slot(void* cache, int* slot);
int friday_cache_free_slot(void* cache, int slot);
int friday_cache_reserve(void* cache, int n, const int* slots, const int* q_lens);
int friday_cache_commit(void* cache, int n, const int* slots, const int* q_lens);
int friday_cache_info(void* cache, const char** json);

/* the generation loop alone, with the step function and the sampler handed in */
typedef struct FridayLoopHooks {
    void* user;
    int (*step)(void* user, int n, const int* slots, const int* token_offsets, const int* tokens, const int* want_offsets,
                const int* want);
    int (*sample)(void* user, int n, const int* streams, const int* steps, int* out);
    int (*alloc_slot)(void* user, int* slot);
    int (*free_slot)(void* user, int slot);
} FridayLoopHooks;
int friday_generate_loop(int n_prompts, const int* offsets, const int* tokens, const FridayLoopHooks* hooks, int max_batch,
                         int max_context, int vocab_size, const char* options_json, const char** result_json);

/* the engine */
int friday_engine_new(const char* options_json, void** engine);
void friday_engine_free(void* engine);
int friday_engine_info(void* engine, const char** json);
int friday_engine_alloc_slot(void* engine, int* slot);
int friday_engine_free_slot(void* engine, int slot);
int friday_engine_slot_length(void* engine, int slot, int* length);
int friday_engine_step(void* engine, int n, const int* slots, const int* token_offsets, const int* tokens,
                       const int* want_offsets, const int* want, float* logits, int logits_on_device, int64_t* rows);
int friday_engine_step_token(void* engine, int token, int pos, float* logits);
int friday_engine_prefill(void* engine, const int* tokens, int n, int pos, float* logits);
typedef void (*friday_on_step)(void* user, int n, const int* requests, const int* tokens);
int friday_engine_generate(void* engine, int n_prompts, const int* offsets, const int* tokens, const char* options_json,
                           friday_on_step on_step, void* user, const char** result_json);
/* the next `launches` tensor-core products write their CTAs' time stamps to trace[launch][sm][16] (uint64) */
int friday_engine_set_trace(void* engine, void* trace, int launches);
int friday_engine_check(void* engine);
int friday_engine_profile(void* engine, const char** json);
int friday_engine_stats(void* engine, const char** json);

int friday_decoder_new(void* engine, int n, const int* slots, const int* first_tokens, float temperature, uint64_t seed,
                       const int* streams, const int* steps_done, void** decoder);
int friday_decoder_step(void* decoder, const int* tokens);
int friday_decoder_sampled(void* decoder, int* out);
int friday_decoder_logits(void* decoder, float* out, int on_device);
int friday_decoder_retire(void* decoder, int row);
int friday_decoder_info(void* decoder, const char** json);
int friday_decoder_close(void* engine, void* decoder);          /* hands it back to the engine, which keeps it */
void friday_decoder_free(void* decoder);

/* the operations, for tests of the kernels and measurements; results go to tensors the caller provides */
int friday_ops_new(int device, void* stream, void** ops);
void friday_ops_free(void* ops);
int friday_ops_embedding(void* ops, const int* tokens, int64_t n, const FridayTensor* table, FridayTensor* out);
int friday_ops_gather_rows(void* ops, const int* rows, int64_t n, const FridayTensor* src, FridayTensor* out);
int friday_ops_rmsnorm(void* ops, const FridayTensor* x, const FridayTensor* weight, float eps, FridayTensor* out);
int friday_ops_swiglu(void* ops, const FridayTensor* gate_up, FridayTensor* out);
int friday_ops_rope_kv_write(void* ops, FridayTensor* qkv, const int* row_seq, const int* row_pos, const float* denominators,
                             int rotary_dim, int n_heads, int n_kv_heads, int head_dim, const FridayKV* kv);
int friday_ops_advance(void* ops, int* tokens, const int* sampled, int* row_pos, int* kv_len, const int* row_seq, int* draws,
                       int n);
int friday_ops_scale_rows(void* ops, FridayTensor* x, float scale);
int friday_ops_finish_logits(void* ops, FridayTensor* logits, const FridayTensor* bias, float scale, float softcap);
/* x may come with the first half of an RMSNorm done (ssq non-null): see friday::Rows */
int friday_ops_linear(void* ops, const FridayTensor* x, const FridayTensor* ssq, float eps, const FridayTensor* source,
                      const FridayTensor* norm_weight, const FridayTensor* weight, const FridayTensor* bias,
                      const FridayTensor* residual, FridayTensor* out);
int friday_ops_linear_tc(void* ops, const FridayTensor* x, const FridayTensor* weight, const FridayTensor* bias,
                         const FridayTensor* residual, FridayTensor* out, int swap, int bn, int splits, int act);
int friday_ops_linear_simt(void* ops, const FridayTensor* x, const FridayTensor* weight, const FridayTensor* bias,
                           const FridayTensor* residual, FridayTensor* out);
/* out, normed: [rows, n]; ssq: room for [max_parts, rows] floats.  *deferred: 1 if `normed` holds weight (*) out and
 * ssq the partial sums (ssq->shape[0] is set to the number of parts), 0 if `normed` is the finished norm. */
int friday_ops_linear_norm(void* ops, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                           const FridayTensor* weight, const FridayTensor* norm_weight, float eps, const FridayTensor* bias,
                           const FridayTensor* residual, FridayTensor* out, FridayTensor* normed, FridayTensor* ssq,
                           int* deferred);
int friday_ops_qkv_rope_write(void* ops, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                              const FridayTensor* weight, const FridayTensor* bias, const int* row_seq, const int* row_pos,
                              const float* denominators, int rotary_dim, int n_heads, int n_kv_heads, int head_dim,
                              const FridayKV* kv, FridayTensor* out);
int friday_ops_linear_swiglu(void* ops, const FridayTensor* x, const FridayTensor* in_ssq, float in_eps,
                             const FridayTensor* weight_pairs, FridayTensor* out);
int friday_ops_attention(void* ops, const FridayTensor* q, int64_t q_stride, FridayTensor* out, const FridayKV* kv,
                         const FridayGeometry* geometry, int n_heads, int n_kv_heads, int head_dim, int window, float scale);
int friday_ops_sample(void* ops, const FridayTensor* logits, const float* temperature, const int* streams, const int* steps,
                      uint64_t seed, const int* row_live, int* out);
int friday_ops_plan(void* ops, int64_t rows, int64_t n, int64_t k, int* swapped, int* bn, int* splits);
int friday_ops_decode_splits(void* ops, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int max_kv_len, int* splits);
int friday_ops_attention_splits(void* ops, int64_t rows, int n_heads, int max_kv_len, int* splits);
int friday_ops_tensor_core_ok(void* ops, const FridayTensor* x, const FridayTensor* weight, const FridayTensor* out, int* ok);
int friday_ops_info(void* ops, const char** json);          /* sm_count, fusion, launches, status word address */
int friday_ops_check_status(void* ops);

#ifdef __cplusplus
}
#endif
