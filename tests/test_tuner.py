"""Host-side parts of the tuner: the categorical TPE sampler, constraint pruning, output parsing,
journal resume and the table entry it emits (no GPU: the timing step is replaced by a synthetic cost)."""
import json
import math
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))

from rocm_sgemm_b200.config import tune  # noqa: E402


def synthetic_cost(c):
    """Lower is better; minimum at a known configuration."""
    cost = 1.0
    cost += abs(math.log2(c["block_m"]) - 7) + abs(math.log2(c["block_n"]) - 7) + abs(math.log2(c["block_k"]) - 5) * 0.5
    cost += 0.0 if c["pipeline"] == 1 else 1.0
    cost += 0.0 if c["fma_mode"] == 1 else 0.5
    cost += 0.1 * abs(c["split_k"] - 1)
    return cost


def test_sampler_only_proposes_valid_untried_configurations():
    tpe = tune.CategoricalTPE(tune.SPACE, seed=1, n_startup=5)
    seen = set()
    for _ in range(40):
        c = tpe.ask(tune.valid)
        assert c is not None and tune.valid(c)
        key = tuple(sorted(c.items()))
        assert key not in seen
        seen.add(key)
        tpe.tell(c, synthetic_cost(c))


def test_tpe_beats_random_search_on_a_synthetic_cost():
    def run(n_startup, trials=80, seed=3):
        tpe = tune.CategoricalTPE(tune.SPACE, seed=seed, n_startup=n_startup)
        for _ in range(trials):
            c = tpe.ask(tune.valid)
            tpe.tell(c, synthetic_cost(c))
        return min(v for _, v in tpe.obs)
    guided = sum(run(10, seed=s) for s in range(5)) / 5
    blind = sum(run(10 ** 9, seed=s) for s in range(5)) / 5  # never leaves the random start-up phase
    assert guided <= blind


def test_failed_trials_count_as_bad():
    tpe = tune.CategoricalTPE(tune.SPACE, seed=0, n_startup=2)
    for _ in range(6):
        c = tpe.ask(tune.valid)
        tpe.tell(c, math.inf if c["pipeline"] == 0 else synthetic_cost(c))
    assert tpe.ask(tune.valid) is not None


def test_parse_time():
    assert tune.parse_time("manual_time 2.125000 ms min 2.101000 ms tflops 64.7\n") == (2.125, 2.101)
    assert tune.parse_time("CUDA error") is None


def test_entry_schema_and_searched_entry_properties():
    cfg = dict(zip(tune.NAMES, tune.BASELINES[0][0]), split_k=2, pretranspose=3)
    e = tune.entry((4096, 4096, 4096), (0, 1, 0), cfg)
    assert e["range"] == {"M": 4096, "N": 4096, "K": 4096}
    assert e["layout"] == {"A": "row_major", "B": "col_major", "C": "row_major"}
    assert e["config"]["split_k"] == 2 and e["config"]["pretranspose"] == 3
    assert tune.gc.check_variant(tune.gc.variant_of(e["config"])) is None
    # pre-transposition is a searched property: only bits of K-contiguous operands are valid for a layout
    assert tune.valid(cfg, (0, 1, 0)) and not tune.valid(cfg, (1, 1, 0)) and not tune.valid(cfg, (1, 0, 0))
    assert tune.valid(dict(cfg, pretranspose=2), (1, 1, 0)) and tune.valid(dict(cfg, pretranspose=0), (1, 0, 0))
    # split_k 0 (equal K ranges per CTA) belongs to the warp-specialised kernel only
    assert tune.valid(dict(cfg, split_k=0, pretranspose=0), (0, 0, 0))
    assert not tune.valid(dict(cfg, split_k=0, pretranspose=0, pipeline=0, fma_mode=2), (0, 0, 0))


def test_max_memory_bound():
    cfg = dict(zip(tune.NAMES, tune.BASELINES[0][0]), split_k=1, pretranspose=0)
    need = tune.smem_bytes(cfg)
    assert need == 4 * (128 + 128) * 32 * 4 + (2 * 4 + 4) * 8 + 16
    assert tune.valid(cfg, (1, 0, 0), max_memory=need) and not tune.valid(cfg, (1, 0, 0), max_memory=need - 1)
    # a K-contiguous operand that is not pre-transposed adds the staging ring
    assert tune.smem_bytes(cfg, (0, 0, 0)) == need + 1024 + 2 * 128 * 128


def test_multivariate_sampler_follows_joint_structure():
    """A cost whose optimum needs two parameters to agree (block_m == block_n): the multivariate sampler reaches it
    at least as well as the independent one on average."""
    def cost(c):
        return 1.0 + (0.0 if c["block_m"] == c["block_n"] else 1.0) + 0.2 * abs(math.log2(c["block_k"]) - 5) \
            + (0.0 if c["pipeline"] == 1 else 0.5)

    def run(multivariate, seed, trials=60):
        tpe = tune.CategoricalTPE(tune.SPACE, seed=seed, n_startup=10, multivariate=multivariate)
        for _ in range(trials):
            c = tpe.ask(tune.valid)
            tpe.tell(c, cost(c))
        good = sorted(v for _, v in tpe.obs)[:10]
        return sum(good) / len(good)
    joint = sum(run(True, s) for s in range(6)) / 6
    indep = sum(run(False, s) for s in range(6)) / 6
    assert joint <= indep + 0.05


def test_resume_from_journal(tmp_path, monkeypatch):
    calls = []

    def fake_time(cands, shape, layout, workdir, iters=20, timeout=60):
        calls.append(len(cands))
        return [synthetic_cost(c) for c in cands]

    monkeypatch.setattr(tune, "time_candidates", fake_time)
    journal = tmp_path / "j.jsonl"
    best1 = tune.tune_problem((512, 512, 512), (0, 0, 0), 12, 7, journal, tmp_path, batch=4, seeds=tune.BASELINES[:2])
    assert len(journal.read_text().splitlines()) == 12
    n_calls = len(calls)
    # same budget again: everything is replayed from the journal, nothing is timed
    best2 = tune.tune_problem((512, 512, 512), (0, 0, 0), 12, 7, journal, tmp_path, batch=4)
    assert len(calls) == n_calls and best2[1] == best1[1]
    # a larger budget continues from there
    tune.tune_problem((512, 512, 512), (0, 0, 0), 16, 7, journal, tmp_path, batch=4)
    assert len(journal.read_text().splitlines()) == 16
    recs = [json.loads(l) for l in journal.read_text().splitlines()]
    assert all(r["shape"] == [512, 512, 512] and r["layout"] == [0, 0, 0] for r in recs)
