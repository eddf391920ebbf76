/* Plain C user of the public header: proves that include/nfai_cuda.h is valid C and that the library links and runs
 * without Python. Host-only calls (version, tokenizer); with a GPU present (argv[1] = "gpu") it also creates and
 * destroys a context. Prints "ok" and returns 0 on success. */
#include <stdio.h>
#include <string.h>

#include "nfai_cuda.h"

int main(int argc, char** argv) {
  if (!nfai_version() || !nfai_version()[0]) return 1;
  const char* tokens[] = {"<|eot_id|>", "a", "b", "ab", "\xC4\xA0", "\xC4\xA0" "ab"};
  const uint32_t token_lens[] = {10, 1, 1, 2, 2, 4};
  const char* merges[] = {"a b", "\xC4\xA0 ab"};
  const uint32_t merge_lens[] = {3, 5};
  nfai_tokenizer* t = NULL;
  if (nfai_tokenizer_create(tokens, token_lens, 6, merges, merge_lens, 2, 0, 0, &t) != NFAI_OK) return 2;
  uint32_t ids[16];
  size_t n = 0;
  const char* text = "<|eot_id|>ab ab";
  if (nfai_tokenizer_encode(t, text, strlen(text), ids, 16, &n) != NFAI_OK) return 3;
  if (n != 3 || ids[0] != 0 || ids[1] != 3 || ids[2] != 5) return 4;
  char out[64];
  size_t m = 0;
  if (nfai_tokenizer_decode(t, ids, n, out, sizeof out, &m) != NFAI_OK) return 5;
  if (m != strlen(text) || memcmp(out, text, m) != 0) return 6;
  if (nfai_tokenizer_encode(t, "<|nope|>x", 9, ids, 16, &n) == NFAI_OK) return 7; /* unknown special token */
  nfai_tokenizer_destroy(t);
  if (argc > 1 && strcmp(argv[1], "gpu") == 0) {
    nfai_ctx* c = NULL;
    if (nfai_ctx_create(0, &c) != NFAI_OK) return 8;
    nfai_ctx_destroy(c);
  }
  printf("ok %s\n", nfai_version());
  return 0;
}
