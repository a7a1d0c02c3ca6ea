/* C interface of the reflex_b200 engine.
 *
 * In the manner of the reference's include/reflex_engine.h (opaque model handle,
 * int status with 0 = success and -1 = failure, a thread-local last error with a
 * stable numeric category, result buffers owned by the library and released by
 * NULL-safe, idempotent free functions; include/reflex_engine.h:46-73, 155-214,
 * 260-328).  Where the reference takes text and owns a tokenizer, this library
 * takes token ids.
 *
 * The engine's host side is Python; this library runs it in an interpreter
 * inside the calling process (started at the first call unless the process
 * already runs one).  No Python exception crosses this boundary: every failure
 * is returned as a status and recorded for rfx_last_error().  A handle is not
 * thread-safe: use it from one thread at a time.
 */
#ifndef REFLEX_B200_H
#define REFLEX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Categories of rfx_last_error_code(); values never change meaning
 * (src/error.rs:72-90 of the reference). */
typedef enum {
    RFX_CODE_OK = 0,
    RFX_CODE_CHECKPOINT = 1,
    RFX_CODE_UNSUPPORTED_ARCHITECTURE = 2,
    RFX_CODE_CUDA = 3,
    RFX_CODE_CUBLAS = 4,
    RFX_CODE_OUT_OF_MEMORY = 5,
    RFX_CODE_TOKENIZER = 6,
    RFX_CODE_CONTEXT_OVERFLOW = 7,
    RFX_CODE_KV_CACHE = 8,
    RFX_CODE_LORA = 9,
    RFX_CODE_IO = 10,
    RFX_CODE_INVALID_INPUT = 11,
    RFX_CODE_OTHER = 12,
    RFX_CODE_PANIC = 13,
    RFX_CODE_GRAMMAR_DEAD_END = 14
} RfxErrorCode;

typedef struct RfxModel RfxModel;

/* Sampling options with the reference's meanings (src/sampling.rs:36-66):
 * temperature <= 0 is greedy; top_k 0 and top_p outside (0, 1) are off;
 * seed < 0 draws a seed from the system. */
typedef struct {
    float temperature;
    int32_t top_k;
    float top_p;
    int64_t seed;
    const uint32_t *stop_token_ids;
    size_t num_stop_token_ids;
} RfxSampling;

typedef struct {
    uint32_t *token_ids;
    size_t num_tokens;
} RfxSequence;

typedef struct {
    RfxSequence *sequences; /* one per prompt, in the prompts' order */
    size_t num_sequences;
} RfxGenerateResult;

typedef struct {
    float score;       /* sum of the raw head logits of the candidate's tokens */
    float probability; /* softmax of the scores over the temperature */
} RfxCandidateScore;

typedef struct {
    RfxCandidateScore *candidates;
    size_t num_candidates;
    size_t best_idx;
    float entropy; /* bits */
} RfxScoreResult;

typedef struct {
    float *logits; /* [rows, vocab], rows in the order of the entries and of their wanted places */
    size_t rows;
    size_t vocab;
} RfxStepResult;

/* One request's share of a step: its next tokens and the places among them
 * whose logits are wanted. */
typedef struct {
    int64_t sequence; /* from rfx_open_sequence */
    const uint32_t *tokens;
    size_t num_tokens;
    const uint32_t *want;
    size_t num_want;
} RfxStepEntry;

/* Message and category of the last failure on this thread; NULL and
 * RFX_CODE_OK after a call that succeeded.  The string is valid until the next
 * call into the library on this thread. */
const char *rfx_last_error(void);
RfxErrorCode rfx_last_error_code(void);

/* model_dir: a folder with config.json and model.safetensors.  weights: "bf16"
 * (NULL means this) or "f32".  max_tokens: the most tokens live sequences hold
 * (each rounded up to a multiple of 64); 0 takes the default.  max_batch: most
 * sequences of one batch; 0 takes the default.  NULL on failure. */
RfxModel *rfx_load(const char *model_dir, const char *weights, size_t max_tokens, size_t max_batch);

/* Writes a model folder with random weights from a config.json file and a
 * seed into out_dir, then loads it. */
RfxModel *rfx_load_random(const char *config_json, uint64_t seed, const char *out_dir,
                          const char *weights, size_t max_tokens, size_t max_batch);

void rfx_free(RfxModel *model);

/* Generates up to max_new_tokens (at least 1) for every prompt; a stop token is
 * kept in the output and ends its sequence.  sampling NULL is greedy. */
int rfx_generate(RfxModel *model, const uint32_t *const *prompts, const size_t *prompt_lens,
                 size_t num_prompts, size_t max_new_tokens, const RfxSampling *sampling,
                 RfxGenerateResult *out);
void rfx_free_generate_result(RfxGenerateResult *result);

/* Scores continuations of one prompt in a single prefill step. */
int rfx_score(RfxModel *model, const uint32_t *prompt, size_t prompt_len,
              const uint32_t *const *candidates, const size_t *candidate_lens,
              size_t num_candidates, float temperature, RfxScoreResult *out);
void rfx_free_score_result(RfxScoreResult *result);

/* The step function itself.  A sequence is opened, stepped with its prompt
 * (together with others that start in the same step), stepped one token at a
 * time, and closed, which gives back what it holds. */
int rfx_open_sequence(RfxModel *model, int64_t *sequence);
int rfx_close_sequence(RfxModel *model, int64_t sequence);
int rfx_step(RfxModel *model, const RfxStepEntry *entries, size_t num_entries, RfxStepResult *out);
void rfx_free_step_result(RfxStepResult *result);

#ifdef __cplusplus
}
#endif
#endif /* REFLEX_B200_H */
