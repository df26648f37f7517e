/* Drives the C API from a plain C program (no Python on the host side): errors as results, generation loop, tokenizer and
 * stream, tensors, the continuous-batching engine, handle accounting, shutdown and use after shutdown.
 * Behaviour checked against the reference's C API tests (test/c_api_tests.cpp: error results, GreedySearch loops, engine
 * loops).  Usage: c_api_test <model_dir>; prints `key: value` lines that the pytest wrapper compares with the Python API. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ogb_genai_c.h"

#define CHECK(call)                                                          \
  do {                                                                       \
    OgaResult* r_ = (call);                                                  \
    if (r_) {                                                                \
      fprintf(stderr, "FAILED %s: %s\n", #call, OgaResultGetError(r_));      \
      OgaDestroyResult(r_);                                                  \
      exit(1);                                                               \
    }                                                                        \
  } while (0)

static void print_tokens(const char* key, const int32_t* t, size_t n) {
  printf("%s:", key);
  for (size_t i = 0; i < n; ++i) printf(" %d", t[i]);
  printf("\n");
}

static int n_log_lines = 0;
static void on_log(const char* s, size_t n) { (void)s; (void)n; ++n_log_lines; }

static void generate(const char* dir, int max_length, const char* key) {
  OgaModel* model; OgaTokenizer* tok; OgaSequences* seqs; OgaGeneratorParams* params; OgaGenerator* gen;
  CHECK(OgaCreateModel(dir, &model));
  CHECK(OgaCreateTokenizer(model, &tok));
  CHECK(OgaCreateSequences(&seqs));
  CHECK(OgaTokenizerEncode(tok, "hello world", seqs));
  CHECK(OgaCreateGeneratorParams(model, &params));
  CHECK(OgaGeneratorParamsSetSearchNumber(params, "max_length", max_length));
  CHECK(OgaGeneratorParamsSetSearchBool(params, "do_sample", false));
  CHECK(OgaCreateGenerator(model, params, &gen));
  CHECK(OgaGenerator_AppendTokenSequences(gen, seqs));
  while (!OgaGenerator_IsDone(gen)) CHECK(OgaGenerator_GenerateNextToken(gen));
  print_tokens(key, OgaGenerator_GetSequenceData(gen, 0), OgaGenerator_GetSequenceCount(gen, 0));
  OgaDestroyGenerator(gen); OgaDestroyGeneratorParams(params); OgaDestroySequences(seqs); OgaDestroyTokenizer(tok); OgaDestroyModel(model);
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  const char* dir = argv[1];

  /* errors come back as results, and the library stays usable */
  OgaModel* bad = NULL;
  OgaResult* err = OgaCreateModel("/nonexistent/model/dir", &bad);
  printf("bad_model_error: %s\n", err ? "yes" : "no");
  if (err) OgaDestroyResult(err);

  CHECK(OgaSetLogCallback(on_log));
  CHECK(OgaSetLogBool("enabled", false));

  OgaModel* model; OgaTokenizer* tok; OgaSequences* seqs; OgaGeneratorParams* params; OgaGenerator* gen;
  CHECK(OgaCreateModel(dir, &model));
  const char* type;
  CHECK(OgaModelGetType(model, &type));
  printf("model_type: %s\n", type);
  OgaDestroyString(type);
  CHECK(OgaCreateTokenizer(model, &tok));
  CHECK(OgaCreateSequences(&seqs));
  CHECK(OgaTokenizerEncode(tok, "hello world", seqs));
  print_tokens("prompt", OgaSequencesGetSequenceData(seqs, 0), OgaSequencesGetSequenceCount(seqs, 0));

  CHECK(OgaCreateGeneratorParams(model, &params));
  CHECK(OgaGeneratorParamsSetSearchNumber(params, "max_length", 24));
  CHECK(OgaGeneratorParamsSetSearchBool(params, "do_sample", false));
  double ml = 0;
  CHECK(OgaGeneratorParamsGetSearchNumber(params, "max_length", &ml));
  printf("max_length: %d\n", (int)ml);
  err = OgaGeneratorParamsSetSearchNumber(params, "no_such_option", 1);
  printf("bad_option_error: %s\n", err ? "yes" : "no");
  if (err) OgaDestroyResult(err);

  CHECK(OgaCreateGenerator(model, params, &gen));
  CHECK(OgaGenerator_AppendTokenSequences(gen, seqs));
  OgaTokenizerStream* stream;
  CHECK(OgaCreateTokenizerStream(tok, &stream));
  char streamed[4096] = "";
  for (size_t i = 0; i < OgaSequencesGetSequenceCount(seqs, 0); ++i) {
    const char* piece;
    CHECK(OgaTokenizerStreamDecode(stream, OgaSequencesGetSequenceData(seqs, 0)[i], &piece));
    strncat(streamed, piece, sizeof(streamed) - strlen(streamed) - 1);
  }
  printf("streamed_prompt: %s\n", streamed);
  size_t n_generated = 0;
  while (!OgaGenerator_IsDone(gen)) {
    CHECK(OgaGenerator_GenerateNextToken(gen));
    const int32_t* next; size_t n_next;
    CHECK(OgaGenerator_GetNextTokens(gen, &next, &n_next));
    n_generated += n_next;
  }
  printf("generated: %zu\n", n_generated);
  size_t n_seq = OgaGenerator_GetSequenceCount(gen, 0);
  const int32_t* seq = OgaGenerator_GetSequenceData(gen, 0);
  print_tokens("greedy", seq, n_seq);
  printf("token_count: %zu\n", OgaGenerator_TokenCount(gen));
  size_t n_prompt = OgaSequencesGetSequenceCount(seqs, 0);
  const char* text;
  CHECK(OgaTokenizerDecode(tok, seq, n_prompt, &text));
  printf("decoded_prompt: %s\n", text);
  OgaDestroyString(text);

  /* logits as a tensor: [1, 1, vocab] float32 */
  OgaTensor* logits;
  CHECK(OgaGenerator_GetLogits(gen, &logits));
  size_t rank; int64_t shape[3]; OgaElementType et;
  CHECK(OgaTensorGetShapeRank(logits, &rank));
  CHECK(OgaTensorGetShape(logits, shape, rank));
  CHECK(OgaTensorGetType(logits, &et));
  printf("logits: rank %zu rows %d type %d\n", rank, (int)shape[0], (int)et);
  OgaDestroyTensor(logits);

  /* rewind and regenerate: same continuation */
  CHECK(OgaGenerator_RewindTo(gen, n_prompt));
  while (!OgaGenerator_IsDone(gen)) CHECK(OgaGenerator_GenerateNextToken(gen));
  print_tokens("after_rewind", OgaGenerator_GetSequenceData(gen, 0), OgaGenerator_GetSequenceCount(gen, 0));
  OgaDestroyTokenizerStream(stream);
  OgaDestroyGenerator(gen);

  /* caller-owned tensor memory and named tensors */
  float data[6] = {1, 2, 3, 4, 5, 6};
  int64_t dims[2] = {2, 3};
  OgaTensor* t; OgaNamedTensors* named; OgaTensor* back; void* ptr; size_t count;
  CHECK(OgaCreateTensorFromBuffer(data, dims, 2, OgaElementType_float32, &t));
  CHECK(OgaCreateNamedTensors(&named));
  CHECK(OgaNamedTensorsSet(named, "x", t));
  CHECK(OgaNamedTensorsCount(named, &count));
  CHECK(OgaNamedTensorsGet(named, "x", &back));
  CHECK(OgaTensorGetData(back, &ptr));
  printf("named_tensors: %zu value %.0f\n", count, ((float*)ptr)[5]);
  OgaDestroyTensor(back); OgaDestroyTensor(t); OgaDestroyNamedTensors(named);

  /* continuous batching: two requests through the engine */
  OgaEngine* engine;
  CHECK(OgaCreateEngine(model, &engine));
  OgaRequest* reqs[2];
  int32_t out[2][64]; size_t n_out[2] = {0, 0};
  long tags[2] = {0, 1};
  const char* prompts[2] = {"hello world", "The quick brown fox"};
  for (int i = 0; i < 2; ++i) {
    OgaSequences* s;
    CHECK(OgaCreateSequences(&s));
    CHECK(OgaTokenizerEncode(tok, prompts[i], s));
    CHECK(OgaCreateRequest(params, &reqs[i]));
    CHECK(OgaRequestAddTokens(reqs[i], s));
    CHECK(OgaRequestSetOpaqueData(reqs[i], &tags[i]));
    CHECK(OgaEngineAddRequest(engine, reqs[i]));
    OgaDestroySequences(s);
  }
  bool pending = true;
  int guard = 0;
  while (pending && guard++ < 1000) {
    OgaRequest* ready = NULL;
    CHECK(OgaEngineStep(engine, &ready));
    if (ready) {
      void* tag; bool unseen = false;
      CHECK(OgaRequestGetOpaqueData(ready, &tag));
      long id = *(long*)tag;
      CHECK(OgaRequestHasUnseenTokens(ready, &unseen));
      while (unseen && n_out[id] < 64) {
        CHECK(OgaRequestGetUnseenToken(ready, &out[id][n_out[id]++]));
        CHECK(OgaRequestHasUnseenTokens(ready, &unseen));
      }
      OgaDestroyRequest(ready);
    }
    CHECK(OgaEngineHasPendingRequests(engine, &pending));
  }
  for (int i = 0; i < 2; ++i) {
    bool unseen = false, complete = false;
    CHECK(OgaRequestHasUnseenTokens(reqs[i], &unseen));
    while (unseen && n_out[i] < 64) {
      CHECK(OgaRequestGetUnseenToken(reqs[i], &out[i][n_out[i]++]));
      CHECK(OgaRequestHasUnseenTokens(reqs[i], &unseen));
    }
    CHECK(OgaRequestIsTurnComplete(reqs[i], &complete));
    printf("engine_complete_%d: %s\n", i, complete ? "yes" : "no");
    CHECK(OgaEngineRemoveRequest(engine, reqs[i]));
    OgaDestroyRequest(reqs[i]);
  }
  print_tokens("engine_0", out[0], n_out[0]);
  print_tokens("engine_1", out[1], n_out[1]);
  OgaDestroyEngine(engine);

  OgaDestroyGeneratorParams(params); OgaDestroySequences(seqs); OgaDestroyTokenizer(tok); OgaDestroyModel(model);
  printf("live_before_shutdown: %zu\n", OgaLiveHandleCount());
  OgaShutdown();

  /* the library is usable again after a shutdown */
  generate(dir, 16, "after_shutdown");

  /* a handle that is never destroyed is reported by the next shutdown */
  OgaSequences* leaked;
  CHECK(OgaCreateSequences(&leaked));
  printf("live_with_leak: %zu\n", OgaLiveHandleCount());
  fflush(stdout);
  OgaShutdown();
  return 0;
}
