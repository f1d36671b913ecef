/* Public C ABI of the engine (libb200infer.so).
 *
 * A thin, language-neutral surface over the Python engine: model load happens on first use,
 * requests and results are JSON documents with the same field names as the engine's request
 * records (TextRequest, ImageRequest, VideoRequest, ModelSpec, EngineOptions), tokens stream
 * through a callback. The .NET facade (dotnet/HartsyInference.B200) P/Invokes exactly these
 * functions and keeps the reference's public types (InferenceEngine, ModelSpec, TextRequest,
 * ImageRequest; reference: src/HartsyInference.Engine/Services/IInferenceEngine.cs:6-45).
 *
 * Every function returns 0 on success or a positive error code (see b200_error_code in
 * exceptions.py: 1 generic, 2 out of device memory, 3 unsupported model, 4 unsupported backend,
 * 5 KV pool exhausted, 6 queue full, 7 native library, 8 device wait timeout, 9 communication,
 * 10 cancelled); b200_last_error() returns the message of the last failure on this thread.
 * Strings returned through out-parameters are owned by the caller and released with b200_free().
 */
#ifndef B200INFER_H_
#define B200INFER_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_engine b200_engine;

/* kind: "chunk" | "result" | "status" | "stop_reason"; payload: UTF-8 text or JSON. Return non-zero
 * from the callback to cancel the request. */
typedef int (*b200_chunk_cb)(const char* kind, const char* payload, void* user);
/* step / total of a denoise loop; return non-zero to cancel. */
typedef int (*b200_step_cb)(int step, int total, void* user);

int b200_engine_create(const char* backend_selector, const char* options_json, b200_engine** out);
void b200_engine_destroy(b200_engine* e);
int b200_engine_set_backend(b200_engine* e, const char* backend_selector);
int b200_engine_describe(b200_engine* e, char** json_out);
int b200_engine_is_supported(b200_engine* e, const char* modality);
int b200_free_memory(b200_engine* e);

int b200_text_generate(b200_engine* e, const char* spec_json, const char* request_json, char** result_json_out);
int b200_text_stream(b200_engine* e, const char* spec_json, const char* request_json, b200_chunk_cb cb, void* user);
int b200_text_count_tokens(b200_engine* e, const char* spec_json, const char* request_json, int* tokens_out);

/* rgb_out: width * height * 3 bytes (RGB24), released with b200_free(). */
int b200_image_generate(b200_engine* e, const char* spec_json, const char* request_json, b200_step_cb cb, void* user,
                        uint8_t** rgb_out, int* width, int* height, long long* seed);
/* frames_out: frame_count * width * height * 3 bytes, frames back to back. */
int b200_video_generate(b200_engine* e, const char* spec_json, const char* request_json, b200_step_cb cb, void* user,
                        uint8_t** frames_out, int* frame_count, int* width, int* height, int* fps, long long* seed);

/* Speech to text. pcm: mono float samples in [-1, 1] at sample_rate Hz. result_json_out: {"text", "language",
   "duration", "segments": [{"start", "end", "text"}]}; released with b200_free(). */
int b200_transcribe(b200_engine* e, const char* spec_json, const char* request_json, const float* pcm, long long samples,
                    int sample_rate, char** result_json_out);
/* Text to speech. pcm_out: mono float samples, released with b200_free(). */
int b200_speak(b200_engine* e, const char* spec_json, const char* request_json, float** pcm_out, long long* samples_out,
               int* sample_rate_out);
/* Text to music. request_json: {"prompt", "seconds", "guidance", "greedy", "seed"}. pcm_out: mono float samples, released with b200_free(). */
int b200_music(b200_engine* e, const char* spec_json, const char* request_json, float** pcm_out, long long* samples_out,
               int* sample_rate_out);
/* Text embeddings. texts_json: a JSON array of strings. out: count * dim floats (row-major), released with b200_free(). */
int b200_embed_text(b200_engine* e, const char* spec_json, const char* texts_json, float** out, int* count, int* dim);
/* Image embedding of one RGB24 image. out: dim floats (L2-normalised), released with b200_free(). */
int b200_embed_image(b200_engine* e, const char* spec_json, const uint8_t* rgb, int width, int height, float** out, int* dim);
/* Upscale one RGB24 image. rgb_out: width_out * height_out * 3 bytes, released with b200_free(). */
int b200_upscale(b200_engine* e, const char* spec_json, const char* request_json, const uint8_t* rgb, int width, int height,
                 uint8_t** rgb_out, int* width_out, int* height_out);

const char* b200_last_error(void);
void b200_free(void* p);
const char* b200_version(void);

#ifdef __cplusplus
}
#endif
#endif
