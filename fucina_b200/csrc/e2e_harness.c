/* A C caller of the blocking and the asynchronous host-buffer entry points, for timing without an interpreter
 * between the calls: the Q4_K decode stack (K = 4096 -> N in {4096, 11008, 4096, 32000}) at batch m, host
 * activations in, host results out, resident weights. Weights are synthetic but well-formed Q4_K blocks (f16
 * scales of 0.01 / 0.005, random 6-bit scale bytes and nibbles): timing does not depend on the values.
 * Prints one JSON line. Built next to the library; links only libdl.
 *
 *   e2e_harness [m] [steps] [library path]
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct fq_work fq_work;
typedef int (*init_fn)(int);
typedef int (*gemm_fn)(int, const void*, size_t, int, size_t, const float*, float*, size_t, size_t, size_t);
typedef int (*async_fn)(int, const void*, size_t, int, size_t, size_t, const float*, fq_work*, float*, size_t, size_t, size_t, size_t, fq_work**);
typedef int (*finish_fn)(fq_work*, int);
typedef void (*destroy_fn)(fq_work*);
typedef int (*sync_fn)(void);
typedef int (*reg_fn)(void*, size_t);
typedef int (*err_fn)(char*, size_t);

static double now_s(void) {
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

int main(int argc, char** argv) {
    const int m = argc > 1 ? atoi(argv[1]) : 1;
    const int steps = argc > 2 ? atoi(argv[2]) : 300;
    const char* path = argc > 3 ? argv[3] : NULL;
    char def[4096];
    if (!path) {
        /* the library sits beside this binary */
        ssize_t n = readlink("/proc/self/exe", def, sizeof def - 32);
        if (n <= 0) return 2;
        def[n] = 0;
        char* slash = strrchr(def, '/');
        strcpy(slash ? slash + 1 : def, "libfucina_b200.so");
        path = def;
    }
    void* h = dlopen(path, RTLD_NOW);
    if (!h) {
        fprintf(stderr, "dlopen: %s\n", dlerror());
        return 2;
    }
    init_fn fq_init = (init_fn)dlsym(h, "fq_init");
    gemm_fn fq_gemm = (gemm_fn)dlsym(h, "fq_gemm_quant_nt");
    async_fn fq_async = (async_fn)dlsym(h, "fq_gemm_quant_nt_async");
    finish_fn fq_finish = (finish_fn)dlsym(h, "fq_work_finish");
    destroy_fn fq_destroy = (destroy_fn)dlsym(h, "fq_work_destroy");
    sync_fn fq_sync = (sync_fn)dlsym(h, "fq_synchronize");
    reg_fn fq_reg = (reg_fn)dlsym(h, "fq_host_register");
    err_fn fq_err = (err_fn)dlsym(h, "fq_last_error");
    if (!fq_init || !fq_gemm || !fq_async || !fq_finish || !fq_destroy || !fq_sync || !fq_reg || !fq_err) return 2;
    if (fq_init(-1) != 0) {
        char buf[256];
        fq_err(buf, sizeof buf);
        printf("{\"error\": \"fq_init: %s\"}\n", buf);
        return 0;
    }
    enum { K = 4096, NP = 4, COPIES = 5, Q4_K = 2 };
    static const size_t N[NP] = {4096, 11008, 4096, 32000};
    const size_t row_bytes = K / 256 * 144;
    uint8_t* w[COPIES][NP];
    uint32_t seed = 12345u;
    for (int c = 0; c < COPIES; ++c)
        for (int p = 0; p < NP; ++p) {
            const size_t bytes = N[p] * row_bytes;
            uint8_t* b = (uint8_t*)malloc(bytes);
            if (!b) return 2;
            for (size_t i = 0; i < bytes; i += 4) {
                seed = seed * 1664525u + 1013904223u;
                memcpy(b + i, &seed, 4);
            }
            for (size_t blk = 0; blk < bytes; blk += 144) {
                b[blk] = 0x1f, b[blk + 1] = 0x21; /* d    = f16 0.01  */
                b[blk + 2] = 0x1f, b[blk + 3] = 0x1d; /* dmin = f16 0.005 */
            }
            w[c][p] = b;
        }
    float* x[NP];
    float* y[NP];
    float* xr[NP];
    float* yr[NP];
    size_t h2d = 0, d2h = 0, wbytes = 0;
    for (int p = 0; p < NP; ++p) {
        x[p] = (float*)malloc(sizeof(float) * m * K);
        y[p] = (float*)malloc(sizeof(float) * m * N[p]);
        xr[p] = (float*)aligned_alloc(4096, (sizeof(float) * m * K + 4095) & ~(size_t)4095);
        yr[p] = (float*)aligned_alloc(4096, (sizeof(float) * m * N[p] + 4095) & ~(size_t)4095);
        for (size_t i = 0; i < (size_t)m * K; ++i) {
            seed = seed * 1664525u + 1013904223u;
            x[p][i] = xr[p][i] = (float)((int)(seed >> 8) % 2001 - 1000) * 1e-3f;
        }
        h2d += sizeof(float) * m * K, d2h += sizeof(float) * m * N[p];
        wbytes += N[p] * row_bytes;
    }
    const double bytes_step = (double)(wbytes + h2d + d2h);
    int rc = 0;
    /* first touch adopts every copy's weights */
    for (int c = 0; c < COPIES && rc == 0; ++c)
        for (int p = 0; p < NP && rc == 0; ++p) rc = fq_gemm(Q4_K, w[c][p], N[p] * row_bytes, 1, row_bytes, x[p], y[p], m, N[p], K);
    if (rc != 0) {
        char buf[256];
        fq_err(buf, sizeof buf);
        printf("{\"error\": \"warm-up call returned %d: %s\"}\n", rc, buf);
        return 0;
    }
    double t_block, t_async, t_block_reg, t_async_reg, t_submit = 0.0;
    for (int pass = 0; pass < 2; ++pass) {
        float** xi = pass ? xr : x;
        float** yo = pass ? yr : y;
        if (pass)
            for (int p = 0; p < NP; ++p) {
                fq_reg(xr[p], (sizeof(float) * m * K + 4095) & ~(size_t)4095);
                fq_reg(yr[p], (sizeof(float) * m * N[p] + 4095) & ~(size_t)4095);
            }
        for (int s = 0; s < 20; ++s)
            for (int p = 0; p < NP; ++p) fq_gemm(Q4_K, w[s % COPIES][p], N[p] * row_bytes, 1, row_bytes, xi[p], yo[p], m, N[p], K);
        fq_sync();
        double t0 = now_s();
        for (int s = 0; s < steps; ++s)
            for (int p = 0; p < NP; ++p) rc |= fq_gemm(Q4_K, w[s % COPIES][p], N[p] * row_bytes, 1, row_bytes, xi[p], yo[p], m, N[p], K);
        fq_sync();
        const double tb = (now_s() - t0) / steps;
        t0 = now_s();
        double in_submit = 0.0;
        for (int s = 0; s < steps; ++s) {
            fq_work* wk[NP];
            const double s0 = now_s();
            for (int p = 0; p < NP; ++p)
                rc |= fq_async(Q4_K, w[s % COPIES][p], N[p] * row_bytes, 1, row_bytes, N[p] * row_bytes, xi[p], NULL, yo[p], 1, m, N[p], K, &wk[p]);
            in_submit += now_s() - s0;
            for (int p = 0; p < NP; ++p) {
                rc |= fq_finish(wk[p], 1);
                fq_destroy(wk[p]);
            }
        }
        fq_sync();
        const double ta = (now_s() - t0) / steps;
        t_submit = in_submit / steps; /* host time inside the four submits of a step; the rest is waiting and copy-out */
        if (pass) t_block_reg = tb, t_async_reg = ta;
        else t_block = tb, t_async = ta;
    }
    printf("{\"caller\": \"C harness (no interpreter)\", \"batch\": %d, \"steps\": %d, \"rc\": %d, "
           "\"blocking_ms_per_step\": %.4f, \"blocking_GBps\": %.1f, \"async_queue4_ms_per_step\": %.4f, \"async_queue4_GBps\": %.1f, "
           "\"registered_blocking_ms_per_step\": %.4f, \"registered_blocking_GBps\": %.1f, "
           "\"registered_async_queue4_ms_per_step\": %.4f, \"registered_async_queue4_GBps\": %.1f, "
           "\"registered_async_submit_ms_per_step\": %.4f}\n",
           m, steps, rc, t_block * 1e3, bytes_step / t_block / 1e9, t_async * 1e3, bytes_step / t_async / 1e9, t_block_reg * 1e3,
           bytes_step / t_block_reg / 1e9, t_async_reg * 1e3, bytes_step / t_async_reg / 1e9, t_submit * 1e3);
    return 0;
}
