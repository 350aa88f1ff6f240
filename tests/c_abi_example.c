/*
 * A C caller of libb200ew.so -- no Python, no C++: shows that the boundary is a
 * plain C ABI.  Without a GPU (argv[1] == "nogpu") it only checks that entry
 * points report errors through status codes.  With a GPU it
 *   1. sums 1e6 floats with the fixed-function reduction (caller scratch) and
 *      with the no-allocation variant, twice, and compares with the host sum;
 *   2. instantiates a kernel from source at run time (the path the op-tree
 *      engine uses: NVRTC + cache + launch with one by-value parameter block);
 *   3. transposes a 300 x 500 float matrix with b200_dimshuffle, takes the log2
 *      histogram of its values and runs one Kahan accumulation step on it.
 * Exit status 0 = all checks passed.
 */
#include "b200ew.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CHECK(call)                                                          \
    do {                                                                     \
        b200_status st_ = (call);                                            \
        if (st_ != B200_OK) {                                                \
            char msg[512];                                                   \
            b200_last_error(msg, sizeof msg);                                \
            fprintf(stderr, "%s -> %d: %s\n", #call, (int)st_, msg);         \
            return 1;                                                        \
        }                                                                    \
    } while (0)

static const char *kSource =
    "struct P { unsigned long long x; float a; int n; };\n"
    "extern \"C\" __global__ void scale(const __grid_constant__ P p) {\n"
    "    int i = blockIdx.x * blockDim.x + threadIdx.x;\n"
    "    if (i < p.n) reinterpret_cast<float*>(p.x)[i] *= p.a;\n"
    "}\n";

struct Params { unsigned long long x; float a; int n; };

int main(int argc, char **argv) {
    if (b200_version() < 100) return 1;
    if (argc > 1 && strcmp(argv[1], "nogpu") == 0) {
        uint64_t p = 0;
        if (b200_device_count(NULL) != B200_ERR_INVALID) return 1;
        if (b200_malloc(16, &p) != B200_ERR_INVALID) return 1;       /* b200_init not called */
        if (b200_reduce_full_noalloc(0, B200_F32, 4, B200_SUM, 0, 0, 0) != B200_ERR_INVALID) return 1;
        char msg[256];
        if (b200_last_error(msg, sizeof msg) == 0) return 1;
        printf("C-ABI-NOGPU-OK\n");
        return 0;
    }

    const uint64_t n = 1000000;
    float *host = (float *)malloc(n * sizeof(float));
    double want = 0.0;
    for (uint64_t i = 0; i < n; ++i) { host[i] = (float)((i * 2654435761u) % 1000) / 1000.0f - 0.5f; want += host[i]; }

    CHECK(b200_init(0));
    uint64_t x = 0, out = 0, scratch = 0;
    CHECK(b200_malloc(n * 4, &x));
    CHECK(b200_malloc(4, &out));
    CHECK(b200_malloc(b200_reduce_scratch_bytes(), &scratch));
    CHECK(b200_memset(scratch, 0, 1, b200_reduce_scratch_bytes(), 0));
    CHECK(b200_memcpy_h2d(x, host, n * 4, 0, 1));

    float got = 0.f;
    CHECK(b200_reduce_full(x, B200_F32, n, B200_SUM, 0, out, scratch, 0));
    CHECK(b200_memcpy_d2h(&got, out, 4, 0, 1));
    if (fabs(got - want) > 1e-5 * n * 0.25) { fprintf(stderr, "reduce_full: %g vs %g\n", got, want); return 1; }
    for (int rep = 0; rep < 2; ++rep) {
        float got2 = -1.f;
        CHECK(b200_reduce_full_noalloc(x, B200_F32, n, B200_SUM, 0, out, 0));
        CHECK(b200_memcpy_d2h(&got2, out, 4, 0, 1));
        if (got2 != got) { fprintf(stderr, "noalloc call %d: %g vs %g\n", rep, got2, got); return 1; }
    }

    uint64_t kernel = 0;
    CHECK(b200_kernel_get(kSource, "scale", NULL, 0, &kernel));
    struct Params p;
    memset(&p, 0, sizeof p);
    p.x = x; p.a = 2.0f; p.n = (int)n;
    CHECK(b200_launch(kernel, (uint32_t)((n + 255) / 256), 1, 1, 256, 1, 1, 0, 0, &p, sizeof p, 1, 0));
    CHECK(b200_reduce_full(x, B200_F32, n, B200_SUM, 0, out, scratch, 0));
    CHECK(b200_memcpy_d2h(&got, out, 4, 0, 1));
    if (fabs(got - 2.0 * want) > 1e-5 * n * 0.5) { fprintf(stderr, "after scale: %g vs %g\n", got, 2.0 * want); return 1; }

    /* 3. fixed-function kernels on a 300 x 500 matrix m[r][c] = r + c / 1000 */
    {
        enum { R = 300, C = 500 };
        float *m = (float *)malloc(R * C * sizeof(float)), *t = (float *)malloc(R * C * sizeof(float));
        for (int r = 0; r < R; ++r) for (int c = 0; c < C; ++c) m[r * C + c] = (float)r + (float)c / 1000.0f;
        uint64_t dm = 0, dt = 0, dh = 0, dc = 0;
        CHECK(b200_malloc(R * C * 4, &dm));
        CHECK(b200_malloc(R * C * 4, &dt));
        CHECK(b200_malloc(64 * 4, &dh));
        CHECK(b200_malloc(R * C * 4, &dc));
        CHECK(b200_memcpy_h2d(dm, m, R * C * 4, 0, 1));
        /* output (C, R): output dimension 0 walks the input's columns (stride 1), dimension 1 its rows */
        const int64_t shape[2] = {C, R}, dst_strides[2] = {R, 1}, src_strides[2] = {1, C};
        CHECK(b200_dimshuffle(dt, dm, 4, 2, shape, dst_strides, src_strides, 0));
        CHECK(b200_memcpy_d2h(t, dt, R * C * 4, 0, 1));
        for (int r = 0; r < R; ++r) for (int c = 0; c < C; ++c)
            if (t[c * R + r] != m[r * C + c]) { fprintf(stderr, "dimshuffle at (%d, %d)\n", r, c); return 1; }
        if (b200_dimshuffle(dm, dm, 4, 2, shape, dst_strides, src_strides, 0) != B200_ERR_INVALID) return 1;
        /* histogram: values in [2^k - .., ..) -> bin k + 48; row 0 (values below 0.5) lands in low bins */
        int hist[64], total = 0, top = 0;
        CHECK(b200_log2_hist(dm, B200_F32, R * C, dh, 64, -48, 0));
        CHECK(b200_memcpy_d2h(hist, dh, sizeof hist, 0, 1));
        for (int b = 0; b < 64; ++b) total += hist[b];
        for (int b = 48 + 8; b < 64; ++b) top += hist[b];       /* round(log2 x) >= 8: x >= 2^7.5 = 181.02 */
        if (total != R * C || top != (R - 182) * C + 480) { fprintf(stderr, "hist: %d %d\n", total, top); return 1; }
        /* Kahan step: sum = m, cmp = 0, add = m  ->  sum = 2 m exactly, cmp = 0 */
        CHECK(b200_memset(dc, 0, 4, R * C, 0));
        CHECK(b200_memcpy_d2d(dt, dm, R * C * 4, 0));
        CHECK(b200_compensated_sum(dm, dc, dt, B200_F32, R * C, 1.0f, 1.0f, 0, 0));
        CHECK(b200_memcpy_d2h(t, dm, R * C * 4, 0, 1));
        for (int i = 0; i < R * C; ++i) if (t[i] != 2.0f * m[i]) { fprintf(stderr, "kahan at %d\n", i); return 1; }
        CHECK(b200_free(dm)); CHECK(b200_free(dt)); CHECK(b200_free(dh)); CHECK(b200_free(dc));
        free(m); free(t);
    }

    CHECK(b200_free(x));
    CHECK(b200_free(out));
    CHECK(b200_free(scratch));
    CHECK(b200_shutdown());
    free(host);
    printf("C-ABI-OK sum=%g\n", got);
    return 0;
}
