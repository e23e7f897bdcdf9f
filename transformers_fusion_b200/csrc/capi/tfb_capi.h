/* C API for embedding the framework in a non-Python host program.
 *
 *   quant_model*  quant_model_load(const char* path);       load a .quant checkpoint (+ "<path>.vocab" tokenizer if present)
 *   void          quant_model_free(quant_model*);
 *   char*         quant_generate(quant_model*, const char* prompt, int max_tokens, float temperature, int top_k, float top_p);
 *   void          quant_free_string(char*);
 *   const char*   quant_last_error(void);                    message of the last failed call on this thread ("" if none)
 *
 * The library hosts a CPython interpreter (started on first use, or joined when the caller already runs inside one) and
 * drives the package's inference engine; set TFB_PYTHONPATH to the directory that contains the package when it is not
 * on the default module path.  Calls are serialised by the interpreter lock; strings are UTF-8.
 * Reference counterpart: quant_model_load / quant_model_free / quant_generate / quant_free_string / quant_last_error
 * (include/quant/production.h:140-147). */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

typedef struct quant_model quant_model;

quant_model* quant_model_load(const char* path);
void quant_model_free(quant_model* m);
char* quant_generate(quant_model* m, const char* prompt, int max_tokens, float temperature, int top_k, float top_p);
void quant_free_string(char* s);
const char* quant_last_error(void);

#ifdef __cplusplus
}
#endif
