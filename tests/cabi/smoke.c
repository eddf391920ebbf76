/* Plain C user of the public header: proves that include/nfai_cuda.h is valid C and that the library links and runs
 * without Python. Host-only calls (version, tokenizer). With a GPU present:
 *   smoke gpu                        creates and destroys a context;
 *   smoke gpu <model.gguf> <tokens>  drives the hot path: loads the GGUF file natively, ingests the prompt and decodes
 *                                    greedily on the device; <tokens> is a text file whose first line holds the prompt
 *                                    ids and whose second line holds the tokens that must come out (the first is the
 *                                    arg-max after the prompt, the rest the greedy continuation).
 * Prints "ok" and returns 0 on success. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "nfai_cuda.h"

static int read_ids(FILE* f, uint32_t* out, int cap) {
  char line[1 << 16];
  int n = 0;
  if (!fgets(line, sizeof line, f)) return -1;
  for (char* tok = strtok(line, " \n"); tok && n < cap; tok = strtok(NULL, " \n")) out[n++] = (uint32_t)strtoul(tok, NULL, 10);
  return n;
}

static int hot_path(nfai_ctx* c, const char* gguf, const char* tokens_file) {
  uint32_t prompt[1024], want[1024], got[1024];
  FILE* f = fopen(tokens_file, "r");
  if (!f) return 20;
  const int np = read_ids(f, prompt, 1024), nw = read_ids(f, want, 1024);
  fclose(f);
  if (np < 1 || nw < 2) return 21;
  nfai_hparams probe;
  char why[256];
  if (nfai_gguf_probe(gguf, (uint32_t)(np + nw + 4), &probe, why, sizeof why) != NFAI_OK) {
    fprintf(stderr, "probe: %s\n", why);
    return 22;
  }
  nfai_model* m = NULL;
  if (nfai_model_load_gguf(c, gguf, (uint32_t)(np + nw + 4), -1, &m) != NFAI_OK) {
    fprintf(stderr, "load: %s\n", nfai_last_error(c));
    return 23;
  }
  nfai_hparams hp;
  if (nfai_model_get_hparams(m, &hp) != NFAI_OK || hp.V != probe.V || hp.L != probe.L || hp.H != probe.H) return 24;
  uint32_t am = 0;
  if (nfai_prefill(m, prompt, np, NULL, &am) != NFAI_OK) return 25;
  if (am != want[0]) {
    fprintf(stderr, "arg-max after the prompt: %u, expected %u\n", am, want[0]);
    return 26;
  }
  float ms = 0.f;
  if (nfai_decode_greedy(m, am, nw - 1, got, &ms) != NFAI_OK) return 27;
  for (int i = 0; i < nw - 1; ++i)
    if (got[i] != want[i + 1]) {
      fprintf(stderr, "greedy token %d: %u, expected %u\n", i, got[i], want[i + 1]);
      return 28;
    }
  uint32_t pos = 0;
  if (nfai_position(m, &pos) != NFAI_OK || pos != (uint32_t)(np + nw - 1)) return 29;
  /* a full cache is a status, not an overrun */
  for (int i = 0; i < 8; ++i) {
    int rc = nfai_decode(m, 1, NULL, &am);
    if (rc == NFAI_ERR_CONTEXT_FULL) break;
    if (rc != NFAI_OK || i == 7) return 30;
  }
  nfai_model_destroy(m);
  printf("hot path ok: %d prompt tokens, %d greedy tokens, %.1f us/token\n", np, nw - 1, ms * 1e3f / (float)(nw - 1));
  return 0;
}


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
    if (argc > 3) {
      int rc = hot_path(c, argv[2], argv[3]);
      if (rc) return rc;
    }
    nfai_ctx_destroy(c);
  }
  printf("ok %s\n", nfai_version());
  return 0;
}
