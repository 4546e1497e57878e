/*
 * CPU oracle for the FP32 GEMM path  C[MxN] = A[MxK] * B[KxN].
 *
 * THIS IS TEST INFRASTRUCTURE.  It is a plain-C restatement of the reference's host-side
 * verification GEMM and of the input generators its tests use.  Only the parity tests, the
 * smoke check and the CPU-baseline leg of the benchmark may call it; the product library
 * never links it and has no CPU fallback.
 *
 * Parity status: PINNED.  Every function here is checked against the reference's own
 * unmodified templates (test/test.hpp, common/matrix.hpp) compiled from where they lie into
 * oracle/_ref/ (see oracle/Makefile, oracle/ref_driver.cpp) and against committed fixtures
 * generated from that build (tests/golden/).
 *
 * Layout convention everywhere: 0 = row-major, 1 = col-major
 * (rocm_sgemm/include/rocm_sgemm/kernel/common.hpp:36-40 and common/matrix.hpp:13-17 use the same order).
 * All matrices are packed: a row-major RxC matrix has leading dimension C, a col-major one R
 * (common/matrix.hpp:130-140).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_ROW 0
#define ORACLE_COL 1

/* element (i,j) of a packed rows x cols matrix; follows matrix<T,Layout>::get_index,
 * common/matrix.hpp:130-140 */
static inline size_t idx(int layout, size_t rows, size_t cols, size_t i, size_t j)
{
    return layout == ORACLE_ROW ? i * cols + j : j * rows + i;
}

/* ------------------------------------------------------------------------------------------
 * Input generators
 * ---------------------------------------------------------------------------------------- */

/* 32-bit Mersenne Twister, the published MT19937 algorithm (what std::mt19937 is specified
 * to be); test/test.hpp:15 constructs it with seed 1. */
typedef struct
{
    uint32_t mt[624];
    int      pos;
} oracle_mt19937;

void oracle_mt19937_seed(oracle_mt19937* g, uint32_t seed)
{
    g->mt[0] = seed;
    for(int i = 1; i < 624; ++i)
        g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
    g->pos = 624;
}

uint32_t oracle_mt19937_next(oracle_mt19937* g)
{
    if(g->pos >= 624)
    {
        for(int i = 0; i < 624; ++i)
        {
            uint32_t y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7fffffffu);
            uint32_t v = g->mt[(i + 397) % 624] ^ (y >> 1);
            if(y & 1u)
                v ^= 0x9908b0dfu;
            g->mt[i] = v;
        }
        g->pos = 0;
    }
    uint32_t y = g->mt[g->pos++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9d2c5680u;
    y ^= (y << 15) & 0xefc60000u;
    y ^= y >> 18;
    return y;
}

/* One draw of std::uniform_real_distribution<float>(lo, hi) as GNU libstdc++ evaluates it
 * (the reference is built against libstdc++ on Linux): generate_canonical<float,24> takes a
 * single 32-bit word, converts it to float (round to nearest), divides by 2^32 and clamps a
 * result of 1.0 to the float just below 1; the distribution then returns u*(hi-lo)+lo.
 * Used by init_matrix, test/test.hpp:14-24. */
static inline float uniform_draw(oracle_mt19937* g, float lo, float hi)
{
    float u = (float)oracle_mt19937_next(g) / 4294967296.0f;
    if(u >= 1.0f)
        u = nextafterf(1.0f, 0.0f);
    return u * (hi - lo) + lo;
}

/* Fill a packed rows x cols matrix in logical (row, col) order whatever its layout, exactly as
 * init_matrix does (test/test.hpp:18-24).  The generator state is the caller's, so a caller can
 * either re-seed per matrix (what the reference's tests do: A and B share a stream) or continue
 * one stream from A into B (what the benchmark configurations here do). */
void oracle_fill_uniform(oracle_mt19937* g, int layout, size_t rows, size_t cols, float lo, float hi, float* out)
{
    for(size_t i = 0; i < rows; ++i)
        for(size_t j = 0; j < cols; ++j)
            out[idx(layout, rows, cols, i, j)] = uniform_draw(g, lo, hi);
}

/* Convenience: the reference test's init_matrix, seed 1, U(-1,1) (test/test.hpp:11-25). */
void oracle_init_matrix(int layout, size_t rows, size_t cols, float* out)
{
    oracle_mt19937 g;
    oracle_mt19937_seed(&g, 1u);
    oracle_fill_uniform(&g, layout, rows, cols, -1.0f, 1.0f, out);
}

/* seeded variant: one stream continuing from A (MxK) into B (KxN) */
void oracle_fill_ab(uint32_t seed, int layout_a, int layout_b, size_t M, size_t N, size_t K, float* A, float* B)
{
    oracle_mt19937 g;
    oracle_mt19937_seed(&g, seed);
    oracle_fill_uniform(&g, layout_a, M, K, -1.0f, 1.0f, A);
    if(B)
        oracle_fill_uniform(&g, layout_b, K, N, -1.0f, 1.0f, B);
}

/* The benchmark's cyclic 5-value fill (benchmark/bench.hpp:15-29). */
void oracle_fill_pattern(int layout, size_t rows, size_t cols, float* out)
{
    static const float tmp[5] = {1.025f, 1.05f, 1.075f, 1.1f, 1.0f};
    size_t             l      = 0;
    for(size_t i = 0; i < rows; ++i)
        for(size_t j = 0; j < cols; ++j)
            out[idx(layout, rows, cols, i, j)] = tmp[(l++) % 5];
}

/* K x N identity for the identity-multiply configuration. */
void oracle_fill_identity(int layout, size_t rows, size_t cols, float* out)
{
    memset(out, 0, rows * cols * sizeof(float));
    size_t d = rows < cols ? rows : cols;
    for(size_t i = 0; i < d; ++i)
        out[idx(layout, rows, cols, i, i)] = 1.0f;
}

/* ------------------------------------------------------------------------------------------
 * GEMM restatements.  row_begin/row_end select a band of rows of C so that a bounded sample of a
 * large problem can be evaluated or timed; pass 0, M for the full problem.
 * ---------------------------------------------------------------------------------------- */

/* sgemm_cpu (test/test.hpp:30-45): float accumulator starting at 0, k ascending,
 * acc += A(i,k)*B(k,j) as a separately rounded multiply and add (this file is built with
 * -ffp-contract=off so the compiler cannot fuse them). */
void oracle_sgemm_f32(int lc, int la, int lb, float* C, const float* A, const float* B, size_t M, size_t N, size_t K,
                      size_t row_begin, size_t row_end, int threads)
{
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for(size_t i = row_begin; i < row_end; ++i)
    {
        for(size_t j = 0; j < N; ++j)
        {
            float acc = 0.0f;
            for(size_t k = 0; k < K; ++k)
            {
                float p = A[idx(la, M, K, i, k)] * B[idx(lb, K, N, k, j)];
                acc     = acc + p;
            }
            C[idx(lc, M, N, i, j)] = acc;
        }
    }
}

/* The same loop with each step a single fused multiply-add.  This is what the reference's GPU
 * kernel evaluates (one accumulator per C element, k ascending, `c += a*b` contracted to an FMA:
 * rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:188-266), and what the CUDA kernels here
 * evaluate within one K-slice.  With `splits` > 1 the K range is cut into `splits` contiguous
 * slices of ceil(K/splits) rounded up to a multiple of `k_align`; each slice is an independent
 * FMA chain from zero and the slice sums are added in ascending slice order starting from
 * slice 0's value: the split-K reduction order of the CUDA path. */
void oracle_sgemm_fma(int lc, int la, int lb, float* C, const float* A, const float* B, size_t M, size_t N, size_t K,
                      size_t row_begin, size_t row_end, int splits, size_t k_align, int threads)
{
    if(splits < 1)
        splits = 1;
    if(k_align < 1)
        k_align = 1;
    size_t per = (K + (size_t)splits - 1) / (size_t)splits;
    per        = (per + k_align - 1) / k_align * k_align;
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for(size_t i = row_begin; i < row_end; ++i)
    {
        for(size_t j = 0; j < N; ++j)
        {
            float total = 0.0f;
            for(int s = 0; s < splits; ++s)
            {
                size_t k0 = (size_t)s * per, k1 = k0 + per < K ? k0 + per : K;
                float  acc = 0.0f;
                for(size_t k = k0; k < k1; ++k)
                    acc = fmaf(A[idx(la, M, K, i, k)], B[idx(lb, K, N, k, j)], acc);
                total = (s == 0) ? acc : total + acc;
            }
            C[idx(lc, M, N, i, j)] = total;
        }
    }
}

/* The same chains with tile-dependent K cut points (the schedule that cuts the tiles' K extents into equal ranges
 * per CTA): C(i,j) belongs to tile (i / block_m) * ceil(N / block_n) + j / block_n, whose cut points are
 * bounds[offsets[t] .. offsets[t+1]) (ascending, strictly between 0 and K).  Every piece is a k-ascending fmaf chain
 * from zero; the owner of the tile's last piece adds the earlier pieces to its own chain in ascending K order:
 * total = ((p_last + p0) + p1) + ...  (with two pieces that is p0 + p1 either way: float addition commutes).
 * (The reference's kernel, kernel/kernel.hpp:188-266, is the single-piece case.) */
void oracle_sgemm_fma_pieces(int lc, int la, int lb, float* C, const float* A, const float* B, size_t M, size_t N,
                             size_t K, size_t row_begin, size_t row_end, size_t block_m, size_t block_n,
                             const int* offsets, const int* bounds, int threads)
{
    const size_t grid_n = (N + block_n - 1) / block_n;
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for(size_t i = row_begin; i < row_end; ++i)
    {
        for(size_t j = 0; j < N; ++j)
        {
            const size_t t     = (i / block_m) * grid_n + j / block_n;
            const int    first = offsets[t], last = offsets[t + 1];
            /* the last piece first: it is the chain the other pieces are added to */
            float total = 0.0f;
            for(size_t k = last > first ? (size_t)bounds[last - 1] : 0; k < K; ++k)
                total = fmaf(A[idx(la, M, K, i, k)], B[idx(lb, K, N, k, j)], total);
            size_t k0 = 0;
            for(int piece = first; piece < last; ++piece)
            {
                const size_t k1  = (size_t)bounds[piece];
                float        acc = 0.0f;
                for(size_t k = k0; k < k1; ++k)
                    acc = fmaf(A[idx(la, M, K, i, k)], B[idx(lb, K, N, k, j)], acc);
                total += acc;
                k0 = k1;
            }
            C[idx(lc, M, N, i, j)] = total;
        }
    }
}

/* float64 accumulation of the exact float products; the yardstick for the error bound
 * 1e-5*sqrt(K).  Output stays in double. */
void oracle_sgemm_f64(int lc, int la, int lb, double* C, const float* A, const float* B, size_t M, size_t N, size_t K,
                      size_t row_begin, size_t row_end, int threads)
{
#ifdef _OPENMP
#pragma omp parallel for num_threads(threads > 0 ? threads : 1) schedule(static)
#endif
    for(size_t i = row_begin; i < row_end; ++i)
    {
        for(size_t j = 0; j < N; ++j)
        {
            double acc = 0.0;
            for(size_t k = 0; k < K; ++k)
                acc += (double)A[idx(la, M, K, i, k)] * (double)B[idx(lb, K, N, k, j)];
            C[idx(lc, M, N, i, j)] = acc;
        }
    }
}

/* Error metrics of a float result against a float64 reference over rows [row_begin,row_end).
 *   out[0] = max |c - ref|
 *   out[1] = max |c - ref| / max(|ref|, rms(ref))      (the relative error the tolerance is stated on)
 *   out[2] = rms(ref) over the band
 *   out[3] = rms(c - ref) over the band
 * Both matrices are indexed with layout lc. */
void oracle_error_metrics(int lc, const float* C, const double* ref, size_t M, size_t N, size_t row_begin,
                          size_t row_end, double* out)
{
    double ss = 0.0;
    size_t n  = 0;
    for(size_t i = row_begin; i < row_end; ++i)
        for(size_t j = 0; j < N; ++j)
        {
            double r = ref[idx(lc, M, N, i, j)];
            ss += r * r;
            ++n;
        }
    double rms     = n ? sqrt(ss / (double)n) : 0.0;
    double max_abs = 0.0, max_rel = 0.0, se = 0.0;
    for(size_t i = row_begin; i < row_end; ++i)
        for(size_t j = 0; j < N; ++j)
        {
            size_t p = idx(lc, M, N, i, j);
            double d = fabs((double)C[p] - ref[p]);
            se += d * d;
            double s = fabs(ref[p]) > rms ? fabs(ref[p]) : rms;
            if(d > max_abs)
                max_abs = d;
            if(s > 0.0 && d / s > max_rel)
                max_rel = d / s;
        }
    out[0] = max_abs;
    out[1] = max_rel;
    out[2] = rms;
    out[3] = n ? sqrt(se / (double)n) : 0.0;
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
