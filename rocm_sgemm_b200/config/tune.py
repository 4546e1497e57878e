#!/usr/bin/env python3
"""TPE tuner for the B200 SGEMM kernel variants.

The counterpart of the reference's rocm_sgemm/config/tune.py (OptunaTuner, :16-374; CLI :531-711): for
every (problem size, A/B/C layout) a Tree-structured Parzen Estimator search over categorical tile
parameters, constraint pruning that does not consume budget (:100-144, :210-212), seeding with baseline
configurations or the entry of an existing table (:261-279), one process per timed trial with a timeout
(:163-190), and a merged output JSON in the table's schema (:650-671).  Differences:

  * Optuna is not a dependency: the sampler below is a small categorical TPE.  Good / bad split at the best
    25 %; by default MULTIVARIATE like the reference's study (tune.py:248-256, multivariate=True): l(x) and g(x) are
    Parzen mixtures with one component per observation (a product of per-parameter categorical kernels that keep
    the observed value with probability 1 - eps), so combinations that work together are proposed together;
    `--independent` falls back to per-parameter Laplace-smoothed frequencies.  The candidate maximising l(x)/g(x)
    among `n_ei_candidates` draws from l is tried next.
  * The search space is the CUDA one: the reference's nine tile parameters plus stages, fma_mode,
    raster, pipeline (kernel variant) and split_k, pretranspose (table entry: split_k 0 = equal K ranges per
    CTA summed inside the kernel; pretranspose bit 0 / 1 = copy a K-contiguous A / B transposed first).  Trials
    run through b200_sgemm_trial, i.e. the drop-in entry's own path.
  * --max-memory bounds the dynamic shared memory of a candidate CTA (the reference's LDS limit flag,
    tune.py:581-582).
  * Candidates are compiled by nvcc a batch at a time into a candidate build of the library
    (rocm_sgemm_b200/build.py), then each is timed by the `tuner` executable in its own process; the
    reference JIT-compiles inside its tuner with hipRTC instead.
  * Every trial is appended to a JSONL journal; a run that is interrupted (or a later run with a larger
    budget) resumes from it.

    python -m rocm_sgemm_b200.config.tune --sizes 4096 --layouts rrr,crr --budget 40 --output tuned.json
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import re
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
sys.path.insert(0, str(HERE))
import generate_config as gc  # noqa: E402

NAMES = list(gc.VARIANT_FIELDS)  # the 14 kernel-variant parameters, in tuple order
SPACE = {
    "block_size": [128, 256],
    "block_m": [64, 128, 256],
    "block_n": [64, 128, 256],
    "block_k": [8, 16, 32, 64],
    "warp_tile_m_count": [1, 2, 4],
    "warp_tile_n_count": [1, 2, 4],
    "thread_tile_m": [4, 8],
    "thread_tile_n": [4, 8],
    "threads_n": [4, 8, 16],
    "stages": [2, 3, 4, 6],
    "fma_mode": [0, 1],
    "raster": [0, 1],
    "min_blocks": [1, 2],
    "pipeline": [0, 1],
    "split_k": [0, 1, 2, 3, 4, 6, 8, 12, 16],
    "pretranspose": [0, 1, 2, 3],
}
ENTRY_KEYS = ("split_k", "pretranspose")  # table-entry properties; the rest are kernel-variant parameters
MAX_SMEM = 227 * 1024
BASELINES = [
    # (14 variant parameters), split_k, pretranspose (masked to the layout's K-contiguous operands)
    ((256, 128, 128, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1), 1, 3),
    ((256, 128, 128, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1), 1, 0),
    ((256, 128, 128, 32, 2, 2, 4, 4, 16, 4, 1, 1, 1, 1), 1, 3),
    ((256, 128, 128, 32, 2, 2, 4, 4, 8, 3, 1, 0, 1, 1), 1, 3),
    ((256, 128, 128, 16, 2, 2, 4, 4, 8, 2, 1, 1, 2, 0), 1, 0),
    ((128, 128, 64, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1), 1, 0),
    ((256, 128, 128, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1), 0, 0),
    ((256, 128, 128, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1), 2, 0),
]
LAYOUT_NAMES = {0: "row_major", 1: "col_major"}


def smem_bytes(cfg: dict, layout=None) -> int:
    """Dynamic shared memory of a candidate CTA: the stage ring, and for the warp-specialised kernel its barriers
    and the staging ring of K-contiguous operands that are not pre-transposed."""
    b = cfg["stages"] * (cfg["block_m"] + cfg["block_n"]) * cfg["block_k"] * 4
    if cfg["pipeline"] >= 1:
        b += (2 * cfg["stages"] + 4) * 8 + 16
        if layout is not None and cfg["block_k"] == 32:
            pre = cfg.get("pretranspose", 0)
            sa = layout[0] == 0 and not (pre & 1)
            sb = layout[1] == 1 and not (pre & 2)
            if sa or sb:
                b += 1024 + 2 * ((cfg["block_m"] * 128 if sa else 0) + (cfg["block_n"] * 128 if sb else 0))
    return b


def valid(cfg: dict, layout=None, max_memory: int = MAX_SMEM) -> bool:
    """Constraint check: the generator's (shared with the build), the table-entry properties, the memory bound."""
    v = tuple(cfg[n] for n in NAMES)
    if gc.check_variant(v) is not None:
        return False
    if cfg["pipeline"] == 0 and cfg["fma_mode"] not in (0, 1, 2):
        return False
    if cfg["split_k"] < 0 or not 0 <= cfg.get("pretranspose", 0) <= 3:
        return False
    if cfg["pipeline"] == 0 and (cfg.get("pretranspose", 0) or cfg["split_k"] == 0):
        return False  # both belong to the warp-specialised kernel
    if layout is not None:
        # only K-contiguous operands can be pre-transposed: other bits would duplicate configurations
        allowed = (1 if layout[0] == 0 else 0) | (2 if layout[1] == 1 else 0)
        if cfg.get("pretranspose", 0) & ~allowed:
            return False
    return smem_bytes(cfg) <= max_memory


def count_valid() -> int:
    """Size of the valid search space (the reference reports 18 060 of 262 144 for its own)."""
    import itertools
    keys = list(SPACE)
    return sum(valid(dict(zip(keys, combo)), (0, 1, 0)) for combo in itertools.product(*(SPACE[k] for k in keys)))


class CategoricalTPE:
    def __init__(self, space, seed=0, gamma=0.25, n_startup=10, n_ei_candidates=24, multivariate=True, eps=0.25):
        self.space, self.rng = space, random.Random(seed)
        self.gamma, self.n_startup, self.n_ei = gamma, n_startup, n_ei_candidates
        self.multivariate, self.eps = multivariate, eps
        self.obs = []  # (cfg, value), lower is better; failed trials carry math.inf

    def tell(self, cfg, value):
        self.obs.append((dict(cfg), value))

    def _random(self):
        return {k: self.rng.choice(v) for k, v in self.space.items()}

    def ask(self, is_valid, max_tries=20000):
        """Next configuration: random during start-up, TPE afterwards; invalid combinations are
        re-drawn without consuming budget, configurations already tried are skipped."""
        seen = {tuple(sorted(c.items())) for c, _ in self.obs}
        finite = [(c, v) for c, v in self.obs if math.isfinite(v)]
        for _ in range(max_tries):
            if len(finite) < self.n_startup:
                cand = self._random()
            else:
                finite.sort(key=lambda cv: cv[1])
                n_good = max(1, int(math.ceil(self.gamma * len(finite))))
                good, bad = [c for c, _ in finite[:n_good]], [c for c, _ in finite[n_good:]] + \
                    [c for c, v in self.obs if not math.isfinite(v)]

                def dist(group, key):
                    w = [1.0 + sum(1 for c in group if c[key] == x) for x in self.space[key]]  # Laplace prior
                    s = sum(w)
                    return [x / s for x in w]

                def mixture(group, c):
                    """Parzen mixture over the observations of `group` plus a uniform prior component."""
                    total = 1.0
                    for key, values in self.space.items():
                        total /= len(values)
                    for o in group:
                        p = 1.0
                        for key, values in self.space.items():
                            p *= (1.0 - self.eps) if c[key] == o[key] else self.eps / max(1, len(values) - 1)
                        total += p
                    return total / (len(group) + 1)

                best, best_score = None, -math.inf
                for _ in range(self.n_ei):
                    c, score = {}, 0.0
                    if self.multivariate:
                        # draw from l: one good observation, each parameter kept with probability 1 - eps
                        o = self.rng.choice(good) if self.rng.random() < len(good) / (len(good) + 1.0) else self._random()
                        for key, values in self.space.items():
                            c[key] = o[key] if self.rng.random() >= self.eps else self.rng.choice(values)
                        score = math.log(mixture(good, c)) - math.log(mixture(bad, c))
                    else:
                        for key, values in self.space.items():
                            pl, pg = dist(good, key), dist(bad, key)
                            i = self.rng.choices(range(len(values)), weights=pl)[0]
                            c[key] = values[i]
                            score += math.log(pl[i]) - math.log(pg[i])
                    if score > best_score and is_valid(c) and tuple(sorted(c.items())) not in seen:
                        best, best_score = c, score
                cand = best or self._random()
            if is_valid(cand) and tuple(sorted(cand.items())) not in seen:
                return cand
        return None


def parse_time(output: str):
    """`manual_time <mean> ms min <min> ms tflops <t>` from the tuner executable."""
    m = re.search(r"manual_time\s+([0-9.eE+-]+)\s+ms\s+min\s+([0-9.eE+-]+)\s+ms", output)
    return (float(m.group(1)), float(m.group(2))) if m else None


def build_tuner_exe(out: Path) -> Path:
    from rocm_sgemm_b200 import build as b
    cmd = [b.nvcc(), "-O2", "-std=c++17", str(HERE / "tuner.cpp"), "-o", str(out), "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=b._env())
    if r.returncode != 0:
        raise RuntimeError(r.stderr)
    return out


def time_candidates(cands, shape, layout, workdir: Path, iters=20, timeout=60):
    """Compile the batch into one candidate library, then one tuner process per candidate."""
    from rocm_sgemm_b200 import build as b
    empty = workdir / "empty.json"
    empty.write_text('{"configurations": []}')
    variants = [tuple(c[n] for n in NAMES) for c in cands]
    lib = workdir / "libcandidate.so"
    pairs = []
    for c, v in zip(cands, variants):
        pre = c.get("pretranspose", 0)
        # a pre-transposed operand reaches the kernel as an M / N-contiguous one: those instantiations are needed too
        for a in {layout[0], 1 if pre & 1 else layout[0]}:
            for bb in {layout[1], 0 if pre & 2 else layout[1]}:
                pairs.append((v, (a, bb, layout[2])))
    try:
        b.build_library(config=empty, extra_pairs=pairs, out=lib)
    except RuntimeError as e:  # one bad candidate fails the batch: fall back to one library per candidate
        if len(cands) == 1:
            return [math.inf]
        return [time_candidates([c], shape, layout, workdir, iters, timeout)[0] for c in cands]
    finally:
        # the shipped library's generated sources were overwritten by the candidate build
        pass
    exe = workdir / "tuner"
    if not exe.exists():
        build_tuner_exe(exe)
    results = []
    for c, v in zip(cands, variants):
        args = [str(exe), str(lib), *map(str, shape), *map(str, v), str(c["split_k"]), str(c.get("pretranspose", 0)),
                *map(str, layout), str(iters), "3"]
        try:
            r = subprocess.run(args, capture_output=True, text=True, timeout=timeout)
            t = parse_time(r.stdout) if r.returncode == 0 else None
        except subprocess.TimeoutExpired:
            t = None
        results.append(t[0] if t else math.inf)
    return results


def tune_problem(shape, layout, budget, seed, journal: Path, workdir: Path, batch=8, seeds=(), multivariate=True,
                 max_memory=MAX_SMEM):
    key = {"shape": list(shape), "layout": list(layout)}
    tpe = CategoricalTPE(SPACE, seed=seed, n_startup=min(10, max(1, budget // 4)), multivariate=multivariate)
    allowed = (1 if layout[0] == 0 else 0) | (2 if layout[1] == 1 else 0)

    def ok(c):
        return valid(c, layout, max_memory)
    # resume: replay the journal
    if journal.exists():
        for line in journal.read_text().splitlines():
            rec = json.loads(line)
            if rec["shape"] == key["shape"] and rec["layout"] == key["layout"] and "pretranspose" in rec["config"]:
                tpe.tell(rec["config"], rec["ms"] if rec["ms"] is not None else math.inf)
    queue = [dict(zip(NAMES, v), split_k=s, pretranspose=p & allowed) for v, s, p in seeds]
    queue = [c for c in queue if ok(c)]
    tried = {tuple(sorted(c.items())) for c, _ in tpe.obs}
    queue = [c for c in queue if tuple(sorted(c.items())) not in tried]
    while len(tpe.obs) < budget:
        cands = []
        while len(cands) < min(batch, budget - len(tpe.obs)):
            c = queue.pop(0) if queue else tpe.ask(ok)
            if c is None:
                break
            if c not in cands:
                cands.append(c)
        if not cands:
            break
        times = time_candidates(cands, shape, layout, workdir)
        with open(journal, "a") as f:
            for c, t in zip(cands, times):
                tpe.tell(c, t)
                f.write(json.dumps({**key, "config": c, "ms": None if not math.isfinite(t) else t}) + "\n")
        best = min(tpe.obs, key=lambda cv: cv[1])
        flops = 2.0 * shape[0] * shape[1] * shape[2]
        print(f"  {len(tpe.obs):3d}/{budget} trials, best {best[1]:.4f} ms = {flops / best[1] / 1e9:.2f} TFLOP/s: {best[0]}",
              flush=True)
    finite = [cv for cv in tpe.obs if math.isfinite(cv[1])]
    return min(finite, key=lambda cv: cv[1]) if finite else None


def entry(shape, layout, cfg):
    conf = {n: cfg[n] for n in NAMES}
    conf["split_k"] = cfg["split_k"]
    conf["pretranspose"] = cfg.get("pretranspose", 0)
    return {"range": dict(zip("MNK", shape)), "layout": {k: LAYOUT_NAMES[x] for k, x in zip("ABC", layout)}, "config": conf}


def load_table(path):
    with open(path) as f:
        return json.load(f)["configurations"]


def table_seed(table, shape, layout):
    for e in table:
        r, l = e["range"], e["layout"]
        if (r["M"], r["N"], r["K"]) == tuple(shape) and tuple(gc.LAYOUT_VAL[l[k]] for k in "ABC") == tuple(layout):
            return [(gc.variant_of(e["config"]), int(e["config"].get("split_k", 1)), int(e["config"].get("pretranspose", 0)))]
    return []


def main():
    ap = argparse.ArgumentParser(description="TPE tuning of the SGEMM kernel variants")
    ap.add_argument("--input", help="existing table: seeds every study and is merged into the output")
    ap.add_argument("--sizes", default="1024,2048,4096,8192", help="cubes M=N=K")
    ap.add_argument("--shapes", default="", help="extra rectangular shapes MxNxK, comma separated")
    ap.add_argument("--layouts", default="all", help="comma separated A,B,C layouts such as rrr,crc; or 'all'")
    ap.add_argument("--baselines", type=int, default=len(BASELINES), help="baseline configurations tried first")
    ap.add_argument("--budget", type=int, default=150, help="trials per (problem, layout)")
    ap.add_argument("--batch", type=int, default=8, help="candidates compiled per build")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--gpu-arch", default="sm_100a", help="kept for the reference's CLI; only sm_100a is built")
    ap.add_argument("--max-memory", type=int, default=MAX_SMEM,
                    help="dynamic shared memory a candidate CTA may use, bytes (default: the 227 KB an SM offers)")
    ap.add_argument("--independent", action="store_true", help="per-parameter TPE instead of the multivariate one")
    ap.add_argument("--journal", default="tune_journal.jsonl")
    ap.add_argument("--output", default="gemm_config_tuned.json")
    ap.add_argument("--count-space", action="store_true", help="print the size of the valid search space and exit")
    a = ap.parse_args()
    if a.count_space:
        total = 1
        for v in SPACE.values():
            total *= len(v)
        print(f"{count_valid()} valid of {total} combinations")
        return
    shapes = [(int(s),) * 3 for s in a.sizes.split(",") if s]
    shapes += [tuple(int(x) for x in s.split("x")) for s in a.shapes.split(",") if s]
    layouts = gc.LAYOUTS if a.layouts == "all" else [tuple("rc".index(ch) for ch in s) for s in a.layouts.split(",")]
    table = load_table(a.input) if a.input else []
    merged = {(e["range"]["M"], e["range"]["N"], e["range"]["K"], e["layout"]["A"], e["layout"]["B"], e["layout"]["C"]): e
              for e in table}
    journal = Path(a.journal)
    with tempfile.TemporaryDirectory() as tmp:
        for shape in shapes:
            for layout in layouts:
                print(f"tuning {shape} layout {gc.layout_str(*layout)}", flush=True)
                seeds = table_seed(table, shape, layout) + BASELINES[:a.baselines]
                best = tune_problem(shape, layout, a.budget, a.seed, journal, Path(tmp), a.batch, seeds,
                                    multivariate=not a.independent, max_memory=a.max_memory)
                if best:
                    e = entry(shape, layout, best[0])
                    merged[(e["range"]["M"], e["range"]["N"], e["range"]["K"], e["layout"]["A"], e["layout"]["B"],
                            e["layout"]["C"])] = e
                    with open(a.output, "w") as f:
                        json.dump({"configurations": list(merged.values())}, f, indent=1)
    # the candidate builds overwrote the generated sources of the shipped library: regenerate them
    from rocm_sgemm_b200 import build as b
    b.generate(b.PKG / "config" / "gemm_config.json")
    print(f"wrote {a.output} ({len(merged)} entries)")


if __name__ == "__main__":
    sys.path.insert(0, str(PKG.parent))
    main()
