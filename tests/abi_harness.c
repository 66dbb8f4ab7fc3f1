/* abi_harness.c -- a plain C caller of libloom_b200.so, the way a cgo or FFI host sees it: includes the public header,
 * links the library, uses host buffers only (loom_b200_dense_forward copies in and out itself).
 *
 *   gcc -std=c99 -Iinclude tests/abi_harness.c -Lloom_b200/lib -lloom_b200 -Wl,-rpath,$PWD/loom_b200/lib -lm -o harness
 *
 * Without a GPU it checks the version and that context creation fails with an error message (exit 0).  With one it
 * runs a 48 x 80 ternary Dense layer on two tokens and compares with the same arithmetic written out in scalar C
 * (absmax int8 quantization with round-half-away, int32 sums over 2-bit codes, float64 rescale: poly/bitnet_cpu.go:46-71,
 * 536-546, 752-776).  Exit status 0 = every output bit matches. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "loom_b200.h"

enum { ROWS = 48, COLS = 80, BATCH = 2 };

static uint32_t lcg(uint32_t* s) { return *s = *s * 1664525u + 1013904223u; }

int main(void) {
    if (loom_b200_api_version() <= 0) {
        fprintf(stderr, "api version %d\n", loom_b200_api_version());
        return 2;
    }
    loom_b200_ctx* ctx = NULL;
    int rc = loom_b200_ctx_create(0, NULL, &ctx);
    if (rc != 0) {
        const char* msg = loom_b200_last_error(NULL);
        printf("no device: rc=%d (%s)\n", rc, msg ? msg : "");
        return (msg && msg[0]) ? 0 : 3; /* an error must come with its message, never with a silent fallback */
    }
    /* ternary weights as the reference packs them: 16 two-bit codes per word, code = weight + 1 */
    const int row_words = (COLS + 15) / 16;
    uint32_t words[ROWS * ((COLS + 15) / 16)];
    int8_t w[ROWS][COLS];
    uint32_t seed = 12345u;
    memset(words, 0, sizeof(words));
    for (int r = 0; r < ROWS; ++r)
        for (int c = 0; c < COLS; ++c) {
            const int t = (int)(lcg(&seed) >> 16) % 3 - 1;
            w[r][c] = (int8_t)t;
            words[r * row_words + c / 16] |= (uint32_t)(t + 1) << (2 * (c % 16));
        }
    for (int r = 0; r < ROWS; ++r) /* tail columns of the last word: code 1 (weight 0), as the reference's packer leaves them */
        for (int c = COLS; c < row_words * 16; ++c) words[r * row_words + c / 16] |= 1u << (2 * (c % 16));
    const float scale = 0.0173f;
    float x[BATCH][COLS], pre[BATCH][ROWS], post[BATCH][ROWS];
    for (int n = 0; n < BATCH; ++n)
        for (int c = 0; c < COLS; ++c) x[n][c] = ((float)(lcg(&seed) >> 8) / 8388608.0f - 1.0f) * 2.5f;

    loom_b200_weight* wt = NULL;
    rc = loom_b200_upload_ternary(ctx, words, ROWS, COLS, row_words, scale, &wt);
    if (rc != 0) {
        fprintf(stderr, "upload_ternary: %d %s\n", rc, loom_b200_last_error(ctx));
        return 4;
    }
    rc = loom_b200_dense_forward(ctx, wt, LOOM_B200_ACT_RELU, &x[0][0], BATCH, &pre[0][0], &post[0][0]);
    if (rc != 0) {
        fprintf(stderr, "dense_forward: %d %s\n", rc, loom_b200_last_error(ctx));
        return 5;
    }
    int bad = 0;
    for (int n = 0; n < BATCH; ++n) {
        float amax = 0.0f;
        for (int c = 0; c < COLS; ++c) amax = fmaxf(amax, fabsf(x[n][c]));
        if (amax < 1e-5f) amax = 1e-5f;
        const double s = 127.0 / (double)amax;
        int q[COLS];
        for (int c = 0; c < COLS; ++c) {
            double v = round((double)x[n][c] * s); /* C's round(): half away from zero, like math.Round */
            if (v > 127.0) v = 127.0;
            if (v < -128.0) v = -128.0;
            q[c] = (int)v;
        }
        const double os = (double)scale * (double)amax / 127.0;
        for (int r = 0; r < ROWS; ++r) {
            int acc = 0;
            for (int c = 0; c < COLS; ++c) acc += (int)w[r][c] * q[c];
            const float want_pre = (float)((double)acc * os);
            const float want_post = want_pre < 0.0f ? 0.0f : want_pre;
            if (memcmp(&want_pre, &pre[n][r], 4) != 0 || memcmp(&want_post, &post[n][r], 4) != 0) {
                if (bad < 5) fprintf(stderr, "token %d row %d: pre %.9g (want %.9g) post %.9g (want %.9g)\n", n, r, pre[n][r], want_pre, post[n][r], want_post);
                ++bad;
            }
        }
    }
    loom_b200_weight_free(ctx, wt);
    loom_b200_ctx_destroy(ctx);
    printf("dense 48x80, 2 tokens: %d of %d outputs differ\n", bad, BATCH * ROWS);
    return bad ? 1 : 0;
}
