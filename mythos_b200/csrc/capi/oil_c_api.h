/* C API of mythos_b200: load a .oil model and generate text from C / C++ / any FFI.
 *
 * The library hosts a CPython interpreter (or joins the one already running in the process) and
 * drives the same engine the Python API uses, so generation runs on the sm_100a kernels. All
 * functions are thread-safe (they take the interpreter lock); errors are reported per thread
 * through oil_last_error(). Mirrors the reference's C API (src/production.cpp:213-372:
 * oil_model_load / oil_model_free / oil_generate / oil_free_string / oil_last_error), except that
 * generation keeps a KV cache instead of re-running the whole prefix for every token.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

typedef struct OilModel OilModel;

/* Returns NULL on failure (see oil_last_error). device: "auto", "cpu", "cuda", "cuda:1", ... */
OilModel* oil_model_load(const char* path);
OilModel* oil_model_load_on(const char* path, const char* device);
void oil_model_free(OilModel* model);

/* Greedy generation. The returned string is heap-allocated; release it with oil_free_string. */
char* oil_generate(OilModel* model, const char* prompt, int max_tokens);
/* Sampling variant: temperature <= 0 means greedy; top_k <= 0 and top_p >= 1 disable the filters. */
char* oil_generate_sampled(OilModel* model, const char* prompt, int max_tokens, float temperature, int top_k,
                           float top_p, unsigned long long seed);
void oil_free_string(char* s);

/* Last error of the calling thread ("" if none). The pointer stays valid until the thread's next call. */
const char* oil_last_error(void);

/* Language / mobile / WASM binding generators of the reference are stubs that log and return false
 * (src/production.cpp:2085-2119); kept as such. */
int oil_generate_binding(const char* language, const char* output_dir);

#ifdef __cplusplus
}
#endif
