// C-linkage doorway onto the REFERENCE's own host code, compiled from where it lies
// (REFERENCE_ROOT/test/test.hpp, REFERENCE_ROOT/common/matrix.hpp) into oracle/_ref/libref_sgemm.so.
// Nothing of the reference is copied: this file only instantiates its templates
//   init_matrix   (test/test.hpp:11-25)
//   sgemm_cpu     (test/test.hpp:30-45)
//   matrix<T,L>   (common/matrix.hpp:24-145)
// for the eight layout permutations and moves data in and out of the matrix objects.
// Test infrastructure only; used to pin oracle/sgemm_oracle.c and to generate tests/golden/.
#include <cstring>
#include <test.hpp>

namespace
{
template<m_layout L>
void do_init(size_t rows, size_t cols, float* out)
{
    matrix<float, L> m(rows, cols);
    init_matrix(m);
    std::memcpy(out, m.data(), rows * cols * sizeof(float));
}

template<m_layout LC, m_layout LA, m_layout LB>
void do_gemm(float* C, const float* A, const float* B, size_t M, size_t N, size_t K)
{
    matrix<float, LA> a(M, K);
    matrix<float, LB> b(K, N);
    matrix<float, LC> c(M, N);
    std::memcpy(a.data(), A, M * K * sizeof(float));
    std::memcpy(b.data(), B, K * N * sizeof(float));
    sgemm_cpu(c, a, b);
    std::memcpy(C, c.data(), M * N * sizeof(float));
}
} // namespace

extern "C" {

// layout: 0 = row-major, 1 = col-major
void ref_init_matrix(int layout, size_t rows, size_t cols, float* out)
{
    if(layout == 0)
        do_init<m_layout::row_major>(rows, cols, out);
    else
        do_init<m_layout::col_major>(rows, cols, out);
}

void ref_sgemm_cpu(int lc, int la, int lb, float* C, const float* A, const float* B, size_t M, size_t N, size_t K)
{
    constexpr m_layout R = m_layout::row_major, Cm = m_layout::col_major;
    switch(la * 4 + lb * 2 + lc)
    {
    case 0: do_gemm<R, R, R>(C, A, B, M, N, K); break;
    case 1: do_gemm<Cm, R, R>(C, A, B, M, N, K); break;
    case 2: do_gemm<R, R, Cm>(C, A, B, M, N, K); break;
    case 3: do_gemm<Cm, R, Cm>(C, A, B, M, N, K); break;
    case 4: do_gemm<R, Cm, R>(C, A, B, M, N, K); break;
    case 5: do_gemm<Cm, Cm, R>(C, A, B, M, N, K); break;
    case 6: do_gemm<R, Cm, Cm>(C, A, B, M, N, K); break;
    default: do_gemm<Cm, Cm, Cm>(C, A, B, M, N, K); break;
    }
}
}
