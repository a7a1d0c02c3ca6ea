/* Drives the engine's C interface the way the reference's ffi-test/smoke_test.c
 * drives its own (ffi-test/smoke_test.c:40-128): failures that need no GPU
 * first, then, given a model folder, generation, scoring and steps.
 *
 *   smoke                      error codes only
 *   smoke MODEL_DIR WEIGHTS    and the GPU paths; prints the tokens and scores
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "reflex_b200.h"

static int expect_code(RfxErrorCode want, const char *what) {
    RfxErrorCode got = rfx_last_error_code();
    if (got != want) {
        fprintf(stderr, "%s: expected code %d, got %d (%s)\n", what, (int)want, (int)got,
                rfx_last_error() ? rfx_last_error() : "no message");
        return 0;
    }
    if (want != RFX_CODE_OK && rfx_last_error() == NULL) {
        fprintf(stderr, "%s: a failure without a message\n", what);
        return 0;
    }
    return 1;
}

int main(int argc, char **argv) {
    /* before any call there is no error */
    if (rfx_last_error() != NULL || rfx_last_error_code() != RFX_CODE_OK) return 1;

    if (rfx_load(NULL, NULL, 0, 0) != NULL || !expect_code(RFX_CODE_INVALID_INPUT, "rfx_load(NULL)")) return 1;
    if (rfx_load("/nonexistent/reflex-b200-model", NULL, 0, 0) != NULL ||
        !expect_code(RFX_CODE_IO, "rfx_load(missing folder)"))
        return 1;
    if (rfx_load_random("/nonexistent/config.json", 1, "/nonexistent/out", NULL, 0, 0) != NULL ||
        !expect_code(RFX_CODE_IO, "rfx_load_random(missing config)"))
        return 1;

    RfxGenerateResult scratch;
    memset(&scratch, 0xff, sizeof scratch);
    if (rfx_generate(NULL, NULL, NULL, 0, 1, NULL, &scratch) != -1 ||
        !expect_code(RFX_CODE_INVALID_INPUT, "rfx_generate(NULL model)"))
        return 1;
    if (scratch.sequences != NULL || scratch.num_sequences != 0) {
        fprintf(stderr, "a failed call must leave a zeroed result\n");
        return 1;
    }
    /* frees take NULL and zeroed structs, twice */
    rfx_free_generate_result(&scratch);
    rfx_free_generate_result(&scratch);
    rfx_free_generate_result(NULL);
    rfx_free_score_result(NULL);
    rfx_free_step_result(NULL);
    rfx_free(NULL);
    printf("RFX_CAPI_ERROR_CODES_OK\n");
    if (argc < 3) return 0;

    RfxModel *model = rfx_load(argv[1], argv[2], 4096, 4);
    if (!model) {
        fprintf(stderr, "rfx_load failed: %s\n", rfx_last_error());
        return 1;
    }
    /* a success clears the earlier failure */
    if (!expect_code(RFX_CODE_OK, "successful rfx_load") || rfx_last_error() != NULL) return 1;

    const uint32_t p0[] = {5, 17, 3, 9}, p1[] = {11, 2};
    const uint32_t *prompts[] = {p0, p1};
    const size_t lens[] = {4, 2};

    if (rfx_generate(model, prompts, lens, 2, 0, NULL, &scratch) != -1 ||
        !expect_code(RFX_CODE_INVALID_INPUT, "max_new_tokens = 0"))
        return 1;
    const uint32_t bad[] = {4000000000u};
    const uint32_t *bad_prompts[] = {bad};
    const size_t one[] = {1};
    if (rfx_generate(model, bad_prompts, one, 1, 1, NULL, &scratch) != -1 ||
        !expect_code(RFX_CODE_INVALID_INPUT, "token outside the vocabulary"))
        return 1;
    /* a prompt longer than any model position */
    size_t too_long = 1u << 20;
    uint32_t *big = calloc(too_long, sizeof *big);
    const uint32_t *big_prompts[] = {big};
    const size_t big_lens[] = {too_long};
    int rc = rfx_generate(model, big_prompts, big_lens, 1, 1, NULL, &scratch);
    free(big);
    if (rc != -1 || !expect_code(RFX_CODE_CONTEXT_OVERFLOW, "over-limit prompt")) return 1;

    RfxGenerateResult gen;
    if (rfx_generate(model, prompts, lens, 2, 6, NULL, &gen) != 0) {
        fprintf(stderr, "rfx_generate failed: %s\n", rfx_last_error());
        return 1;
    }
    if (!expect_code(RFX_CODE_OK, "successful rfx_generate")) return 1;
    for (size_t i = 0; i < gen.num_sequences; i++) {
        printf("RFX_CAPI_GENERATE seq=%zu token_ids=[", i);
        for (size_t j = 0; j < gen.sequences[i].num_tokens; j++)
            printf(j ? ",%u" : "%u", gen.sequences[i].token_ids[j]);
        printf("]\n");
    }

    /* the same through the step function: prompts together, then one token each */
    int64_t s0, s1;
    if (rfx_open_sequence(model, &s0) || rfx_open_sequence(model, &s1)) return 1;
    const uint32_t last0[] = {3}, last1[] = {1};
    RfxStepEntry entries[2] = {{s0, p0, 4, last0, 1}, {s1, p1, 2, last1, 1}};
    RfxStepResult step;
    if (rfx_step(model, entries, 2, &step) != 0 || step.rows != 2) {
        fprintf(stderr, "rfx_step failed: %s\n", rfx_last_error());
        return 1;
    }
    for (size_t r = 0; r < step.rows; r++) {
        size_t best = 0;
        for (size_t v = 0; v < step.vocab; v++)
            if (step.logits[r * step.vocab + v] >= step.logits[r * step.vocab + best]) best = v;
        printf("RFX_CAPI_STEP row=%zu argmax=%zu\n", r, best);
        if ((uint32_t)best != gen.sequences[r].token_ids[0]) {
            fprintf(stderr, "step and generate disagree on the first token of sequence %zu\n", r);
            return 1;
        }
    }
    rfx_free_step_result(&step);
    rfx_free_step_result(&step);
    if (rfx_close_sequence(model, s0) || rfx_close_sequence(model, s1)) return 1;
    if (rfx_close_sequence(model, s0) != -1 || !expect_code(RFX_CODE_KV_CACHE, "a sequence closed twice")) return 1;

    const uint32_t c0[] = {7}, c1[] = {8, 9};
    const uint32_t *cands[] = {c0, c1};
    const size_t clens[] = {1, 2};
    RfxScoreResult sc;
    if (rfx_score(model, p0, 4, cands, clens, 2, 1.0f, &sc) != 0) {
        fprintf(stderr, "rfx_score failed: %s\n", rfx_last_error());
        return 1;
    }
    for (size_t i = 0; i < sc.num_candidates; i++)
        printf("RFX_CAPI_SCORE idx=%zu score=%.6f probability=%.6f\n", i, sc.candidates[i].score,
               sc.candidates[i].probability);
    printf("RFX_CAPI_SCORE_OK best_idx=%zu entropy=%.6f\n", sc.best_idx, sc.entropy);
    rfx_free_score_result(&sc);
    rfx_free_score_result(&sc);

    rfx_free_generate_result(&gen);
    rfx_free_generate_result(&gen);
    rfx_free(model);
    printf("RFX_CAPI_OK\n");
    return 0;
}
