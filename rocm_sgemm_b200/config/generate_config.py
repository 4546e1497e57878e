#!/usr/bin/env python3
"""Build-time code generation for the B200 SGEMM library.

Input: the tuned table `gemm_config.json` — the schema of the reference's
rocm_sgemm/config/gemm_config.json (a list of {range{M,N,K}, layout{A,B,C}, config{...}}) whose
`config` block carries the reference's nine tile parameters plus the optional CUDA-side knobs
`stages`, `fma_mode`, `raster`, `min_blocks`, `pipeline` (kernel-variant properties) and `split_k`,
`pretranspose` (properties of the table entry).

Output, into one directory (the role of rocm_sgemm/config/generate_config.py:7-545):
  config_table.inc        kernel-variant array + sorted (M,N,K,A,B,C) -> (variant, split_k) map
  kernel_inst_v<i>_<abc>.cu   one translation unit per (variant, layout) holding the aligned and the
                          unaligned instantiation (the reference emits one per (config, layout, alignment))
  kernel_lookup.cu        the [variant][layout 0-7][aligned 0/1] kernel table
  sources.txt             the list of generated .cu files for the build step

Only (variant, layout) pairs that appear in the table are instantiated, as in the reference; the
default variant is additionally instantiated for all eight layouts so that a lookup can never land
on an empty slot (in the reference that case throws at run time,
rocm_sgemm/include/rocm_sgemm/kernel_launcher.hpp:89-94).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

NINE = ("block_size", "block_m", "block_n", "block_k", "warp_tile_m_count", "warp_tile_n_count",
        "thread_tile_m", "thread_tile_n", "threads_n")
EXTRA_DEFAULTS = {"stages": 2, "fma_mode": 2, "raster": 1, "min_blocks": 1, "pipeline": 0}
VARIANT_FIELDS = NINE + tuple(EXTRA_DEFAULTS)

# nominal default: 128x128x16 CTA tile, 256 threads, 8x8 per thread as 2x2 sub-tiles of 4x4
DEFAULT_VARIANT = (256, 128, 128, 16, 2, 2, 4, 4, 8, 2, 2, 1, 1, 0)

LAYOUT_VAL = {"row_major": 0, "col_major": 1}
LAYOUTS = [(a, b, c) for a in (0, 1) for b in (0, 1) for c in (0, 1)]  # index = a*4 + b*2 + c
SMEM_LIMIT = 227 * 1024


def layout_str(a: int, b: int, c: int) -> str:
    return "".join("rc"[x] for x in (a, b, c))


def variant_of(cfg: dict) -> tuple:
    return tuple(int(cfg[k]) for k in NINE) + tuple(int(cfg.get(k, d)) for k, d in EXTRA_DEFAULTS.items())


def check_variant(v: tuple) -> str | None:
    """Constraint check shared with the tuner (the reference's is rocm_sgemm/config/tune.py:100-144).
    Returns None when the variant is buildable, else the reason."""
    (bs, bm, bn, bk, wmc, wnc, tm, tn, threads_n, stages, fma_mode, raster, min_blocks, pipeline) = v
    if any(x <= 0 for x in v[:10]) or min_blocks <= 0:
        return "non-positive parameter"
    if 32 % threads_n != 0:
        return "threads_n must divide 32"
    threads_m = 32 // threads_n
    warp_m, warp_n = wmc * tm * threads_m, wnc * tn * threads_n
    if bm % warp_m or bn % warp_n:
        return "warp tile does not divide block tile"
    if (bm // warp_m) * (bn // warp_n) * 32 != bs:
        return "warp grid does not match block_size"
    if bs > 1024:
        return "block_size > 1024"
    if tm not in (1, 2, 4, 8) or tn not in (1, 2, 4, 8):
        return "thread tile must be 1, 2, 4 or 8"
    if bk % 4 or bm % 32 or bn % 32:
        return "block_k % 4, block_m % 32, block_n % 32"
    if stages < 2:
        return "stages < 2"
    if fma_mode not in (0, 1, 2) or raster not in (0, 1, 2):
        return "unknown fma_mode / raster"
    if fma_mode != 0 and tn % 2:
        return "packed FMA needs even thread_tile_n"
    if fma_mode == 2 and tm % 2:
        return "diagonal packing needs even thread_tile_m"
    if pipeline not in (0, 1):
        return "unknown pipeline"
    if stages * (bm + bn) * bk * 4 + (2 * stages * 8 + 16 if pipeline else 0) > SMEM_LIMIT:
        return "shared memory over 227 KB"
    if pipeline >= 1 and fma_mode == 2:
        return "the warp-specialised kernel has no diagonal packing"
    if pipeline >= 1:
        # warp-specialised kernel: 128-bit fragment reads only, TMA boxes of at most 256 elements,
        # consumer warps + one producer warpgroup in one CTA
        if tm not in (4, 8) or tn not in (4, 8):
            return "warp-specialised kernel needs thread tiles of 4 or 8"
        if bm > 256 or bn > 256 or bk > 256:
            return "TMA box dimension over 256"
        producers = 128 if (bs >= 256 and wmc * tm * wnc * tn <= 64) else 64  # ws_producer_threads()
        if bs + producers > 1024:
            return "consumer + producer threads over 1024"
        if (bs + producers) * min_blocks > 2048:
            return "more resident threads than an SM holds"
        if min_blocks * (stages * (bm + bn) * bk * 4 + 2 * stages * 8 + 16) > SMEM_LIMIT:
            return "shared memory of the co-resident CTAs over 227 KB"
    # per-thread accumulators must fit the register file
    if wmc * tm * wnc * tn > 192:
        return "accumulator tile over 192 registers"
    if bs * min_blocks > 2048:
        return "more resident threads than an SM holds"
    return None


def load_table(config_file, extra_variants=()):
    with open(config_file) as f:
        table = json.load(f)
    variants = {DEFAULT_VARIANT} | {tuple(v) for v in extra_variants}
    for conf in table["configurations"]:
        v = variant_of(conf["config"])
        why = check_variant(v)
        if why:
            raise ValueError(f"invalid configuration {v}: {why}")
        variants.add(v)
    variants = sorted(variants)
    entries = {}
    for conf in table["configurations"]:
        r, l = conf["range"], conf["layout"]
        key = (int(r["M"]), int(r["N"]), int(r["K"]), LAYOUT_VAL[l["A"]], LAYOUT_VAL[l["B"]], LAYOUT_VAL[l["C"]])
        entries[key] = (variants.index(variant_of(conf["config"])), int(conf["config"].get("split_k", 1)),
                        int(conf["config"].get("pretranspose", 0)))
    entries = sorted(entries.items())  # by (M, N, K, A, B, C): the order the lookup's binary search needs
    return variants, entries


def needed_pairs(variants, entries):
    pairs = set()
    for key, (vi, _, pre) in entries:
        a, b, c = key[3:6]
        pairs.add((vi, (a, b, c)))
        # a pre-transposed K-contiguous operand is handed to the kernel as an M / N-contiguous one
        if pre:
            pairs.add((vi, (1 if (pre & 1) else a, 0 if (pre & 2) else b, c)))
            pairs.add((vi, (1 if (pre & 1) else a, b, c)))
            pairs.add((vi, (a, 0 if (pre & 2) else b, c)))
    d = variants.index(DEFAULT_VARIANT)
    for lay in LAYOUTS:
        pairs.add((d, lay))
    return sorted(pairs)


def cfg_type(v: tuple) -> str:
    return "TileConfig<" + ", ".join(str(x) for x in v) + ">"


def kernel_header(v: tuple) -> str:
    return "sgemm_ws_kernel.cuh" if v[13] >= 1 else "sgemm_kernel.cuh"


def kernel_name(v: tuple) -> str:
    return "sgemm_ws_kernel" if v[13] >= 1 else "sgemm_kernel"


def generate(config_file, out_dir, extra_pairs=None):
    """extra_pairs: iterable of (variant_tuple, (a,b,c)) to instantiate on top of the table (tuner sweeps)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    extra_pairs = [(tuple(v), tuple(lay)) for v, lay in (extra_pairs or [])]
    for v, _ in extra_pairs:
        why = check_variant(v)
        if why:
            raise ValueError(f"invalid extra variant {v}: {why}")
    variants, entries = load_table(config_file, [v for v, _ in extra_pairs])
    pairs = set(needed_pairs(variants, entries))
    for v, lay in extra_pairs:
        pairs.add((variants.index(v), lay))
    pairs = sorted(pairs)

    # ---- table ------------------------------------------------------------------------------
    lines = ["// Generated by rocm_sgemm_b200/config/generate_config.py - do not edit.",
             f"// {len(variants)} kernel variants, {len(entries)} table entries.",
             f"static constexpr int KERNEL_VARIANTS = {len(variants)};",
             f"static constexpr int DEFAULT_VARIANT_IDX = {variants.index(DEFAULT_VARIANT)};",
             "static const KernelVariant kernel_variants[KERNEL_VARIANTS] = {"]
    for i, v in enumerate(variants):
        lines.append("    {" + ", ".join(str(x) for x in v) + "}, // variant " + str(i))
    lines.append("};")
    lines.append(f"static constexpr int CONFIG_ENTRIES = {len(entries)};")
    lines.append(f"static const ConfigEntry sorted_config_map[{max(1, len(entries))}] = {{")
    for key, (vi, sk, pre) in entries:
        m, n, k, a, b, c = key
        lines.append(f"    {{{{{m}, {n}, {k}, {a}, {b}, {c}}}, {vi}, {sk}, {pre}}}, // {m}x{n}x{k} {layout_str(a, b, c)}")
    if not entries:
        lines.append("    {{0, 0, 0, 0, 0, 0}, 0, 1, 0}")
    lines.append("};")
    (out / "config_table.inc").write_text("\n".join(lines) + "\n")

    # ---- one TU per (variant, layout) ---------------------------------------------------------
    sources = []
    for vi, (a, b, c) in pairs:
        ls = layout_str(a, b, c)
        name = f"kernel_inst_v{vi}_{ls}.cu"
        code = f"""// Generated by rocm_sgemm_b200/config/generate_config.py - do not edit.
// variant {vi}: {dict(zip(VARIANT_FIELDS, variants[vi]))}
// layout A={'row col'.split()[a]} B={'row col'.split()[b]} C={'row col'.split()[c]}
#include "../{kernel_header(variants[vi])}"

namespace sgemm_b200
{{
using Cfg = {cfg_type(variants[vi])};
const void* kernel_v{vi}_{ls}_aligned() {{ return reinterpret_cast<const void*>(&{kernel_name(variants[vi])}<Cfg, {a}, {b}, {c}, true>); }}
const void* kernel_v{vi}_{ls}_unaligned() {{ return reinterpret_cast<const void*>(&{kernel_name(variants[vi])}<Cfg, {a}, {b}, {c}, false>); }}
}} // namespace sgemm_b200
"""
        (out / name).write_text(code)
        sources.append(name)

    # ---- lookup table -------------------------------------------------------------------------
    code = ["// Generated by rocm_sgemm_b200/config/generate_config.py - do not edit.",
            "// kernel table [variant][layout a*4+b*2+c][0 = unaligned, 1 = aligned]; nullptr = not built",
            "#include <cstddef>", "namespace sgemm_b200", "{"]
    for vi, (a, b, c) in pairs:
        ls = layout_str(a, b, c)
        code.append(f"const void* kernel_v{vi}_{ls}_aligned();")
        code.append(f"const void* kernel_v{vi}_{ls}_unaligned();")
    code.append(f"const void* lookup_kernel(int variant, int layout_idx, int aligned)")
    code.append("{")
    code.append(f"    static const void* const table[{len(variants)}][8][2] = {{")
    have = set(pairs)
    for vi in range(len(variants)):
        code.append("        {")
        for (a, b, c) in LAYOUTS:
            ls = layout_str(a, b, c)
            if (vi, (a, b, c)) in have:
                code.append(f"            {{kernel_v{vi}_{ls}_unaligned(), kernel_v{vi}_{ls}_aligned()}},")
            else:
                code.append("            {nullptr, nullptr},")
        code.append("        },")
    code.append("    };")
    code.append(f"    if(variant < 0 || variant >= {len(variants)} || layout_idx < 0 || layout_idx > 7) return nullptr;")
    code.append("    return table[variant][layout_idx][aligned ? 1 : 0];")
    code.append("}")
    code.append("} // namespace sgemm_b200")
    (out / "kernel_lookup.cu").write_text("\n".join(code) + "\n")
    sources.append("kernel_lookup.cu")
    (out / "sources.txt").write_text("\n".join(sources) + "\n")
    return variants, entries, pairs


def main():
    ap = argparse.ArgumentParser(description="Generate the SGEMM configuration table and kernel sources")
    ap.add_argument("config_file")
    ap.add_argument("output_dir")
    args = ap.parse_args()
    variants, entries, pairs = generate(args.config_file, args.output_dir)
    print(f"{len(variants)} variants, {len(entries)} table entries, {len(pairs)} (variant, layout) pairs "
          f"-> {2 * len(pairs)} kernels")


if __name__ == "__main__":
    main()
