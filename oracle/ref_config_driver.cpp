// C-linkage doorway onto the REFERENCE's own configuration selection: the header that the
// reference's generator (rocm_sgemm/config/generate_config.py:7-310) emits from its shipped
// rocm_sgemm/config/gemm_config.json is produced into oracle/_ref/gen/ by oracle/Makefile and
// compiled here, unmodified, for the host.  Test infrastructure only.
#include <rocm_sgemm/kernel/config_generated.hpp>

extern "C" {

int ref_kernel_variants() { return static_cast<int>(rocm_sgemm::KERNEL_VARIANTS); }
int ref_map_entries() { return static_cast<int>(rocm_sgemm::detail::sorted_config_map.size()); }

// find_best_config(M,N,K,layout_A,layout_B,layout_C) -> index into kernel_configs
int ref_find_best_config(size_t m, size_t n, size_t k, int la, int lb, int lc)
{
    using rocm_sgemm::m_layout;
    return static_cast<int>(rocm_sgemm::detail::find_best_config(
        m, n, k, static_cast<m_layout>(la), static_cast<m_layout>(lb), static_cast<m_layout>(lc)));
}

// the nine integers of kernel_configs[idx]
void ref_kernel_config(int idx, int* out)
{
    const auto& c = rocm_sgemm::detail::kernel_configs[idx];
    out[0] = std::get<0>(c); out[1] = std::get<1>(c); out[2] = std::get<2>(c);
    out[3] = std::get<3>(c); out[4] = std::get<4>(c); out[5] = std::get<5>(c);
    out[6] = std::get<6>(c); out[7] = std::get<7>(c); out[8] = std::get<8>(c);
}

// entry i of sorted_config_map: m,n,k,la,lb,lc,config_idx
void ref_map_entry(int i, size_t* out)
{
    const auto& e = rocm_sgemm::detail::sorted_config_map[i];
    out[0] = e.first.m; out[1] = e.first.n; out[2] = e.first.k;
    out[3] = static_cast<size_t>(e.first.layout_a);
    out[4] = static_cast<size_t>(e.first.layout_b);
    out[5] = static_cast<size_t>(e.first.layout_c);
    out[6] = e.second;
}
}
