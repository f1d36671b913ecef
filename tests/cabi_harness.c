/* Stand-alone C program driving the engine through libb200infer.so: create an engine on the CPU
 * backend, generate text from a toy checkpoint (blocking and streaming), generate a tiny image. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "b200infer.h"

static int chunks = 0, got_result = 0, steps = 0;

static int on_chunk(const char* kind, const char* payload, void* user) {
  (void)user;
  if (strcmp(kind, "chunk") == 0) ++chunks;
  if (strcmp(kind, "result") == 0 && strstr(payload, "completion_tokens")) got_result = 1;
  return 0;
}
static int on_step(int step, int total, void* user) { (void)user; (void)total; steps = step; return 0; }

int main(int argc, char** argv) {
  if (argc < 2) { fprintf(stderr, "usage: harness <checkpoint dir>\n"); return 2; }
  b200_engine* e = NULL;
  if (b200_engine_create("cpu", "{\"MaxModelLen\": 256, \"MaxBatch\": 4, \"KvPoolBytesBudget\": 8388608}", &e)) {
    fprintf(stderr, "create: %s\n", b200_last_error());
    return 1;
  }
  if (!b200_engine_is_supported(e, "text") || !b200_engine_is_supported(e, "mesh") || !b200_engine_is_supported(e, "world") || b200_engine_is_supported(e, "fx")) return 3;
  char spec[1024];
  snprintf(spec, sizeof spec, "{\"Requested\": \"%s\", \"Modality\": \"text\", \"LocalPath\": \"%s\"}", argv[1], argv[1]);
  char* result = NULL;
  if (b200_text_generate(e, spec, "{\"Prompt\": \"hello\", \"MaxTokens\": 5, \"Greedy\": true}", &result)) {
    fprintf(stderr, "generate: %s\n", b200_last_error());
    return 4;
  }
  if (!strstr(result, "\"completion_tokens\"")) return 5;
  b200_free(result);
  if (b200_text_stream(e, spec, "{\"Messages\": [{\"role\": \"user\", \"content\": \"hi\"}], \"MaxTokens\": 5, \"Greedy\": true}", on_chunk, NULL)) return 6;
  if (!got_result) return 7;
  int ntok = 0;
  if (b200_text_count_tokens(e, spec, "{\"Prompt\": \"hello\"}", &ntok) || ntok <= 0) return 8;
  unsigned char* rgb = NULL;
  int w = 0, h = 0;
  long long seed = 0;
  if (b200_image_generate(e, "{\"Requested\": \"synthetic:flux-tiny\", \"Modality\": \"image\"}",
                          "{\"Prompt\": \"x\", \"Width\": 64, \"Height\": 64, \"Steps\": 2, \"Seed\": 5}", on_step, NULL, &rgb, &w, &h, &seed)) {
    fprintf(stderr, "image: %s\n", b200_last_error());
    return 9;
  }
  if (w != 64 || h != 64 || seed != 5 || steps != 2 || rgb == NULL) return 10;
  b200_free(rgb);
  if (b200_text_generate(e, "{\"Requested\": \"/no/such\"}", "{}", &result) == 0) return 11;   /* errors come back as codes */
  if (strlen(b200_last_error()) == 0) return 12;
  char* desc = NULL;
  b200_engine_describe(e, &desc);
  printf("CABI_OK chunks=%d tokens=%d %s\n", chunks, ntok, desc ? desc : "");
  b200_free(desc);
  b200_free_memory(e);
  b200_engine_destroy(e);
  return 0;
}
