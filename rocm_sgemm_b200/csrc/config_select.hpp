// Tuned-configuration lookup: (M, N, K, layout_A, layout_B, layout_C) -> table entry.
//
// Same selection rule as the reference's generated detail::find_best_config /
// detail::find_closest_config (rocm_sgemm/config/generate_config.py:173-267):
//   1. exact match by binary search over entries sorted by (m, n, k, layout_a, layout_b, layout_c);
//   2. otherwise the entry with the SAME (A,B,C) layout that minimises
//      (log2 m - log2 m')^2 + (log2 n - log2 n')^2 + (log2 k - log2 k')^2, first minimum in table order;
//   3. otherwise (no entry with that layout) the same distance over all entries;
//   4. an empty table yields -1 and the caller falls back to its default variant.
// Unlike the reference, which bakes the table into constexpr arrays of a generated header, the rule
// lives here as ordinary host code over a caller-supplied table, so it can be unit-tested against any
// table (including the reference's own) without a GPU.  Plain C++17, no CUDA.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <limits>

namespace sgemm_b200
{

// the reference's nine tile parameters (rocm_sgemm/config/gemm_config.json:13-23) plus the
// CUDA-side knobs this implementation adds
struct KernelVariant
{
    int block_size, block_m, block_n, block_k;
    int warp_tile_m_count, warp_tile_n_count, thread_tile_m, thread_tile_n, threads_n;
    int stages, fma_mode, raster, min_blocks, pipeline;
};

struct ConfigKey
{
    size_t m, n, k;
    int    layout_a, layout_b, layout_c; // 0 = row-major, 1 = col-major

    bool operator<(const ConfigKey& o) const
    {
        if(m != o.m) return m < o.m;
        if(n != o.n) return n < o.n;
        if(k != o.k) return k < o.k;
        if(layout_a != o.layout_a) return layout_a < o.layout_a;
        if(layout_b != o.layout_b) return layout_b < o.layout_b;
        return layout_c < o.layout_c;
    }
    bool operator==(const ConfigKey& o) const
    {
        return m == o.m && n == o.n && k == o.k && layout_a == o.layout_a && layout_b == o.layout_b
               && layout_c == o.layout_c;
    }
};

struct ConfigEntry
{
    ConfigKey key;
    int       variant; // index into the kernel-variant array
    int       split_k; // K slices tuned for this problem (1 = none)
    int       pretranspose = 0; // bit 0 / 1: copy a K-contiguous A / B into M / N-contiguous scratch first
};

inline double config_distance(const ConfigKey& a, const ConfigKey& b)
{
    const double dm = std::log2(static_cast<double>(a.m)) - std::log2(static_cast<double>(b.m));
    const double dn = std::log2(static_cast<double>(a.n)) - std::log2(static_cast<double>(b.n));
    const double dk = std::log2(static_cast<double>(a.k)) - std::log2(static_cast<double>(b.k));
    return dm * dm + dn * dn + dk * dk;
}

// steps 2-3; `count` > 0
inline int find_closest_config(const ConfigEntry* map, size_t count, const ConfigKey& target)
{
    double best     = std::numeric_limits<double>::max();
    int    best_idx = -1;
    for(size_t i = 0; i < count; ++i)
    {
        const ConfigKey& key = map[i].key;
        if(key.layout_a == target.layout_a && key.layout_b == target.layout_b && key.layout_c == target.layout_c)
        {
            const double d = config_distance(target, key);
            if(d < best)
            {
                best     = d;
                best_idx = static_cast<int>(i);
            }
        }
    }
    if(best_idx >= 0)
        return best_idx;
    for(size_t i = 0; i < count; ++i)
    {
        const double d = config_distance(target, map[i].key);
        if(d < best)
        {
            best     = d;
            best_idx = static_cast<int>(i);
        }
    }
    return best_idx;
}

// steps 1-4; returns the index of the chosen entry in `map`, or -1 when the table is empty
inline int find_best_config(const ConfigEntry* map, size_t count, const ConfigKey& target)
{
    if(count == 0)
        return -1;
    const ConfigEntry* end = map + count;
    const ConfigEntry* it
        = std::lower_bound(map, end, target, [](const ConfigEntry& e, const ConfigKey& k) { return e.key < k; });
    if(it != end && it->key == target)
        return static_cast<int>(it - map);
    return find_closest_config(map, count, target);
}

// layout index of the dispatch table: rrr=0, rrc=1, rcr=2, rcc=3, crr=4, crc=5, ccr=6, ccc=7
// (rocm_sgemm/include/rocm_sgemm/kernel_launcher.hpp:53-79)
inline int layout_index(int layout_a, int layout_b, int layout_c)
{
    return layout_a * 4 + layout_b * 2 + layout_c;
}

} // namespace sgemm_b200
