/* A host written in C against include/aot_cuda.h only: what a foreign-language binding of
 * the step level does, without any CUDA header or type. Used by the test-suite to check
 * that the header is valid C11, that the library links from C, and (on a GPU) that a model
 * file driven from C gives the tokens and logits the Python binding gets.
 *
 *   client --abi                      print struct sizes and the version; needs no GPU
 *   client <model.bin> <n_ctx> <n_decode> <token> [<token> ...]
 *
 * model.bin = aotcu_model_head, then n_layer x aotcu_layer, then the tensor section
 * (what a generated project holds as CUDA_HEAD, CUDA_LAYERS and the weights blob).
 * Output: one line "tokens: ..." with the greedy continuation, one line "logits: <fnv1a64>"
 * of the final logits' bytes, one line "kv: <fnv1a64> <bytes>" of the saved cache after a
 * save / load round trip into a second Gpu that reproduced the last step. */
#include <inttypes.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "aot_cuda.h"

static uint64_t fnv1a(const void* p, size_t n) {
  const unsigned char* b = (const unsigned char*)p;
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; i++) {
    h ^= b[i];
    h *= 1099511628211ull;
  }
  return h;
}

static int fail(const char* what) {
  fprintf(stderr, "client: %s: %s\n", what, aotcu_last_error());
  return 1;
}

static uint32_t argmax(const float* x, size_t n) { /* first maximum, sampler.rs:99-109 */
  size_t best = 0;
  for (size_t i = 1; i < n; i++)
    if (x[i] > x[best]) best = i;
  return (uint32_t)best;
}

int main(int argc, char** argv) {
  if (argc == 2 && !strcmp(argv[1], "--abi")) {
    printf("version %s\n", aotcu_version());
    printf("sizeof tensor %zu dims %zu layer %zu head %zu\n", sizeof(aotcu_tensor), sizeof(aotcu_dims), sizeof(aotcu_layer),
           sizeof(aotcu_model_head));
    aotcu_ctx* ctx = NULL;
    int rc = aotcu_init(0, &ctx);
    printf("init %d\n", rc);
    if (rc == 0) aotcu_free(ctx);
    return 0;
  }
  if (argc < 5) {
    fprintf(stderr, "usage: client --abi | client <model.bin> <n_ctx> <n_decode> <token>...\n");
    return 2;
  }
  FILE* f = fopen(argv[1], "rb");
  if (!f) {
    perror(argv[1]);
    return 1;
  }
  fseek(f, 0, SEEK_END);
  long size = ftell(f);
  fseek(f, 0, SEEK_SET);
  unsigned char* file = (unsigned char*)malloc((size_t)size);
  if (!file || fread(file, 1, (size_t)size, f) != (size_t)size) {
    fprintf(stderr, "client: cannot read %s\n", argv[1]);
    return 1;
  }
  fclose(f);
  aotcu_model_head head;
  memcpy(&head, file, sizeof head);
  const size_t n_layer = (size_t)head.dims.n_layer;
  aotcu_layer* layers = (aotcu_layer*)malloc(n_layer * sizeof(aotcu_layer));
  memcpy(layers, file + sizeof head, n_layer * sizeof(aotcu_layer));
  const unsigned char* weights = file + sizeof head + n_layer * sizeof(aotcu_layer);
  const size_t weights_len = (size_t)size - (sizeof head + n_layer * sizeof(aotcu_layer));
  const size_t n_ctx = (size_t)atol(argv[2]), n_decode = (size_t)atol(argv[3]), n_prompt = (size_t)(argc - 4);
  const size_t vocab = (size_t)head.dims.vocab;
  uint32_t* toks = (uint32_t*)malloc((n_prompt + n_decode + 1) * sizeof(uint32_t));
  for (size_t i = 0; i < n_prompt; i++) toks[i] = (uint32_t)strtoul(argv[4 + i], NULL, 10);

  aotcu_ctx* ctx = NULL;
  aotcu_gpu *g = NULL, *g2 = NULL;
  if (aotcu_init(0, &ctx)) return fail("aotcu_init");
  if (aotcu_gpu_new(ctx, &head, layers, weights, weights_len, n_ctx, n_prompt, &g)) return fail("aotcu_gpu_new");
  float* logits = (float*)malloc(vocab * sizeof(float));
  if (aotcu_forward_batch(g, toks, n_prompt, 0, 1)) return fail("aotcu_forward_batch");
  if (aotcu_logits(g, logits)) return fail("aotcu_logits");
  size_t n = n_prompt;
  printf("tokens:");
  for (size_t s = 0; s < n_decode; s++) {
    toks[n] = argmax(logits, vocab);
    printf(" %" PRIu32, toks[n]);
    if (aotcu_forward(g, toks[n], n, 1)) return fail("aotcu_forward");
    if (aotcu_logits(g, logits)) return fail("aotcu_logits");
    n++;
  }
  printf("\nlogits: %016" PRIx64 "\n", fnv1a(logits, vocab * sizeof(float)));

  /* save everything but the last position's row, restore into a second Gpu, redo the last step */
  const size_t cap = aotcu_kv_blob_size(g, n, n - 1);
  unsigned char* blob = (unsigned char*)malloc(cap);
  size_t blob_len = 0, got_n = 0, got_cached = 0;
  if (aotcu_kv_save(g, toks, n, n - 1, blob, cap, &blob_len)) return fail("aotcu_kv_save");
  if (aotcu_gpu_new(ctx, &head, layers, weights, weights_len, n_ctx, n_prompt, &g2)) return fail("aotcu_gpu_new (second)");
  uint32_t* back = (uint32_t*)malloc(n * sizeof(uint32_t));
  if (aotcu_kv_load(g2, blob, blob_len, back, n, &got_n, &got_cached)) return fail("aotcu_kv_load");
  if (got_n != n || got_cached != n - 1 || memcmp(back, toks, n * sizeof(uint32_t))) {
    fprintf(stderr, "client: the loaded cache does not describe the saved run\n");
    return 1;
  }
  float* logits2 = (float*)malloc(vocab * sizeof(float));
  if (aotcu_forward(g2, toks[n - 1], n - 1, 1)) return fail("aotcu_forward (restored)");
  if (aotcu_logits(g2, logits2)) return fail("aotcu_logits (restored)");
  if (memcmp(logits, logits2, vocab * sizeof(float))) {
    fprintf(stderr, "client: logits after restoring the cache differ\n");
    return 1;
  }
  printf("kv: %016" PRIx64 " %zu\n", fnv1a(blob, blob_len), blob_len);
  /* a bad call reports an error and leaves the handle usable */
  if (aotcu_forward(g, (uint32_t)vocab, 0, 0) != AOTCU_ERR_BAD_ARG) {
    fprintf(stderr, "client: an out-of-range token was not refused\n");
    return 1;
  }
  aotcu_gpu_free(g2);
  aotcu_gpu_free(g);
  aotcu_free(ctx);
  return 0;
}
