/* Compiled as C99 against include/ternary_b200.h and linked with libternary_b200.so: proves the header is
 * plain C, that every host-side entry point links with C linkage, and runs the host packer end to end.
 * No GPU is touched (device entry points are only called with arguments that validation rejects). */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ternary_b200.h"

int main(void) {
    const int N = 5, K = 32;
    float w[5 * 32];
    for (int i = 0; i < N * K; ++i) w[i] = 0.02f * sinf(0.37f * (float)(i + 1));
    const long long nwords = tbl_packed_words(N, K);
    if (nwords != (N * K + 15) / 16) return 1;
    uint32_t* words = (uint32_t*)calloc((size_t)nwords, sizeof(uint32_t));
    float scale = 0.0f;
    if (tbl_pack_weights(w, N, K, words, &scale) != TBL_OK) return 2;
    /* scale = mean|w| + 1e-8f, codes in {0,1,2} */
    double s = 0.0;
    for (int i = 0; i < N * K; ++i) s += fabs((double)w[i]);
    if (scale != (float)(s / (N * K)) + 1e-8f) return 3;
    int8_t t[5 * 32];
    if (tbl_unpack_weights_i8(words, N, K, t) != TBL_OK) return 4;
    for (int i = 0; i < N * K; ++i) {
        const float v = w[i] / (scale + 1e-8f);
        const int want = v > 0.5f ? 1 : (v < -0.5f ? -1 : 0);
        if (t[i] != want) return 5;
    }
    if (tbl_validate_packed(words, nwords, N, K, scale, NULL, NULL) != TBL_OK) return 6;
    words[0] |= 3u;  /* reserved code */
    if (tbl_validate_packed(words, nwords, N, K, scale, NULL, NULL) != TBL_ERR_CODE) return 7;
    /* device entry points reject bad arguments without touching a GPU */
    if (tbl_linear_forward(NULL, NULL, NULL, NULL, 1.0f, 1, 32, 8, 8, 0, NULL, NULL, NULL, NULL, 0, NULL) != TBL_ERR_INVALID_ARG) return 8;
    if (tbl_linear_workspace_bytes(4, 1024, 8) < 2u * 4u * 1024u) return 9;
    if (tbl_strip_bytes(20, 512) != 32u * 512u / 4u) return 10;
    tbl_linear_view view;
    memset(&view, 0, sizeof view);
    if (sizeof view.strips != sizeof(void*)) return 11;
    if (strcmp(tbl_status_string(TBL_OK), "ok") != 0) return 12;
    free(words);
    printf("abi ok v%d\n", tbl_abi_version());
    return 0;
}
