/*
 * Plain-C restatement of the reference's RNS linear path.  TEST INFRASTRUCTURE
 * ONLY: it checks the CUDA path in tests/ and __graft_entry__.smoke(), and is
 * the timed CPU baseline of bench.py.  Nothing in the product links or calls it.
 *
 * Parity pins: compared in tests/test_oracle.py with the golden vectors under
 * tests/golden/ (outputs of the reference's own NumPy code) and with the NumPy
 * restatement oracle/rns_oracle.py.
 *
 * Stages, each following the reference (paths inside Nek1tt/rns-llm v0.5):
 *   encode   csrc/rns_cuda.cu:98-124        value -> centred residue per channel
 *   gemm     csrc/rns_cuda.cu:478-523       per-channel int8 x int8 -> int32
 *   reduce   csrc/rns_cuda.cu:52-67         canonical residue of each sum
 *   garner   csrc/rns_cuda.cu:380-414       sequential mixed-radix steps
 *   dequant  src/rns_llm/layers/rns_linear.py:264,272-275
 * Deliberately the textbook sequential Garner, not the flattened fp32 form the
 * CUDA epilogue uses, so the two share no arithmetic.
 *
 * Threads: POSIX threads over blocks of output rows; the count is the number
 * of online processors unless RNS_ORACLE_THREADS is set.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#define ORACLE_MAX_CH 10
#define ORACLE_MAX_THREADS 256

int rns_oracle_threads(void) {
    const char* env = getenv("RNS_ORACLE_THREADS");
    long n = env ? atol(env) : sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > ORACLE_MAX_THREADS) n = ORACLE_MAX_THREADS;
    return (int)n;
}

static int64_t inverse_mod(int64_t a, int64_t m) {
    int64_t t = 0, nt = 1, r = m, nr = ((a % m) + m) % m;
    while (nr != 0) {
        int64_t q = r / nr, tmp;
        tmp = t - q * nt; t = nt; nt = tmp;
        tmp = r - q * nr; r = nr; nr = tmp;
    }
    return t < 0 ? t + m : t;
}

static int centred_residue(int v, int m) {
    int r = v % m, half = m / 2;
    if (r > half) r -= m;
    else if (r < -half) r += m;
    return r;
}

/* values int8 [count] -> planes int8 [channels, count] */
void rns_oracle_encode_centered_i8(const int8_t* values, int64_t count, const int32_t* moduli,
                                   int channels, int8_t* planes) {
    for (int c = 0; c < channels; ++c)
        for (int64_t i = 0; i < count; ++i)
            planes[(int64_t)c * count + i] = (int8_t)centred_residue(values[i], moduli[c]);
}

/* sums int32 [channels] of one element -> signed value in (-P/2, P/2] */
static int64_t garner_one(const int32_t* sums, const int32_t* moduli, int channels,
                          const int32_t (*inv)[ORACLE_MAX_CH]) {
    int32_t digit[ORACLE_MAX_CH];
    for (int i = 0; i < channels; ++i) {
        int64_t v = sums[i] % moduli[i];
        if (v < 0) v += moduli[i];
        for (int j = 0; j < i; ++j) {
            v = ((v - digit[j]) * inv[j][i]) % moduli[i];
            if (v < 0) v += moduli[i];
        }
        digit[i] = (int32_t)v;
    }
    int64_t x = 0, place = 1;
    for (int i = 0; i < channels; ++i) { x += place * digit[i]; place *= moduli[i]; }
    if (x > place / 2) x -= place;
    return x;
}

struct linear_job {
    const int8_t *a, *wp;
    int m, n, k, channels, row_begin, row_end;
    const int32_t* moduli;
    const int32_t (*inv)[ORACLE_MAX_CH];
    int64_t* out_i64;
    float* out_f32;
    const float *row_scale, *col_scale, *bias;
    int row_scale_stride;
};

static void* linear_rows(void* arg) {
    const struct linear_job* j = (const struct linear_job*)arg;
    const int k = j->k, n = j->n, channels = j->channels;
    int8_t* ap = (int8_t*)malloc((size_t)channels * k);
    if (!ap) return (void*)1;
    for (int row = j->row_begin; row < j->row_end; ++row) {
        rns_oracle_encode_centered_i8(j->a + (int64_t)row * k, k, j->moduli, channels, ap);
        for (int col = 0; col < n; ++col) {
            int32_t sums[ORACLE_MAX_CH];
            for (int c = 0; c < channels; ++c) {
                const int8_t* ar = ap + (int64_t)c * k;
                const int8_t* wr = j->wp + ((int64_t)c * n + col) * k;
                int32_t s = 0;
                for (int kk = 0; kk < k; ++kk) s += (int32_t)ar[kk] * (int32_t)wr[kk];
                sums[c] = s;
            }
            const int64_t x = garner_one(sums, j->moduli, channels, j->inv);
            const int64_t o = (int64_t)row * n + col;
            if (j->out_i64) j->out_i64[o] = x;
            if (j->out_f32) {
                volatile float y = (float)x;
                y = y * j->row_scale[(int64_t)row * j->row_scale_stride];
                y = y * j->col_scale[col];
                if (j->bias) y = y + j->bias[col];
                j->out_f32[o] = y;
            }
        }
    }
    free(ap);
    return NULL;
}

/*
 * a int8 [M,K] (row stride K), w int8 [N,K] (row stride K): out[m,n] = sum_k a*w
 * through `channels` residue channels.  out_i64 [M,N] may be NULL; out_f32 [M,N]
 * (dequantised, before the cast to the module dtype) may be NULL.
 * row_scale has row_scale_stride 0 (per tensor) or 1 (per row); bias may be NULL.
 * Returns 0, or 1 on a bad argument or failed allocation.
 */
int rns_oracle_linear(const int8_t* a, const int8_t* w, int m, int n, int k,
                      const int32_t* moduli, int channels,
                      int64_t* out_i64, float* out_f32,
                      const float* row_scale, int row_scale_stride,
                      const float* col_scale, const float* bias) {
    if (channels < 1 || channels > ORACLE_MAX_CH || m <= 0 || n <= 0 || k <= 0) return 1;
    int32_t inv[ORACLE_MAX_CH][ORACLE_MAX_CH];
    memset(inv, 0, sizeof(inv));
    for (int i = 0; i < channels; ++i)
        for (int j = 0; j < i; ++j) inv[j][i] = (int32_t)inverse_mod(moduli[j], moduli[i]);

    /* Weight planes once (the reference caches them: backends/cuda_backend.py:464-487). */
    int8_t* wp = (int8_t*)malloc((size_t)channels * n * k);
    if (!wp) return 1;
    rns_oracle_encode_centered_i8(w, (int64_t)n * k, moduli, channels, wp);

    int threads = rns_oracle_threads();
    if (threads > m) threads = m;
    struct linear_job jobs[ORACLE_MAX_THREADS];
    pthread_t tids[ORACLE_MAX_THREADS];
    int failed = 0;
    for (int t = 0; t < threads; ++t) {
        struct linear_job* j = &jobs[t];
        j->a = a; j->wp = wp; j->m = m; j->n = n; j->k = k; j->channels = channels;
        j->row_begin = (int)((int64_t)m * t / threads);
        j->row_end = (int)((int64_t)m * (t + 1) / threads);
        j->moduli = moduli; j->inv = (const int32_t (*)[ORACLE_MAX_CH])inv;
        j->out_i64 = out_i64; j->out_f32 = out_f32;
        j->row_scale = row_scale; j->col_scale = col_scale; j->bias = bias;
        j->row_scale_stride = row_scale_stride;
    }
    if (threads == 1) {
        failed = linear_rows(&jobs[0]) != NULL;
    } else {
        int started = 0;
        for (; started < threads; ++started)
            if (pthread_create(&tids[started], NULL, linear_rows, &jobs[started]) != 0) break;
        for (int t = 0; t < started; ++t) {
            void* rc = NULL;
            pthread_join(tids[t], &rc);
            if (rc != NULL) failed = 1;
        }
        /* rows of threads that could not be started run here */
        for (int t = started; t < threads; ++t)
            if (linear_rows(&jobs[t]) != NULL) failed = 1;
    }
    free(wp);
    return failed;
}

/* sums int32 [channels, count] -> values int64 [count] (Garner only). */
int rns_oracle_garner(const int32_t* sums, int64_t count, const int32_t* moduli, int channels,
                      int64_t* out) {
    if (channels < 1 || channels > ORACLE_MAX_CH) return 1;
    int32_t inv[ORACLE_MAX_CH][ORACLE_MAX_CH];
    memset(inv, 0, sizeof(inv));
    for (int i = 0; i < channels; ++i)
        for (int j = 0; j < i; ++j) inv[j][i] = (int32_t)inverse_mod(moduli[j], moduli[i]);
    for (int64_t e = 0; e < count; ++e) {
        int32_t one[ORACLE_MAX_CH];
        for (int c = 0; c < channels; ++c) one[c] = sums[(int64_t)c * count + e];
        out[e] = garner_one(one, moduli, channels, (const int32_t (*)[ORACLE_MAX_CH])inv);
    }
    return 0;
}
