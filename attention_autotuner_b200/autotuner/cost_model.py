"""Cost model that ranks tile configurations before anything is compiled, so that the search compiles and times only
the most promising few.

The reference planned such a model and never built it: python/tests/export_costmodel_config.py:29-56 exports, per
candidate, the tuple (problem shape, tile shape, MMA shapes, batch, heads) together with the cycle count
python/tests/ncu_profile.py:37-141 scrapes from ncu, and README.md:104 lists the model itself as to do. Here the
training set is what the search already writes: every ``logs/profile_result_*.json`` holds (configuration,
milliseconds) for every candidate that was built and timed on a B200.

Model = analytical features x fitted weights. For a candidate and a problem the features are per-block cycle
budgets derived from the kernel structure (they are what bounds the kernels, see the kernel headers):
  * tensor-pipe cycles executed per (128-row tile, 128-key block), including the recomputation a narrow output
    chunk forces (Q K^T once per chunk of V columns),
  * MUFU cycles of the softmax (one exponential per score, 16 per clock and SM), split by how the tile's softmax is
    organised (one or two query tiles ping-ponging, one or two warpgroups per tile) because those decide how much of
    it hides under the other tile's GEMMs,
  * the share of exponentials moved to the FMA pipes or to packed fp16,
  * the fixed hand-off cost per block (commit -> barrier -> waiting warp), which a deeper ring or a CTA pair changes,
each multiplied by the number of blocks the launch executes and divided by SM count x clock. The weights are a
non-negative least-squares fit of measured milliseconds on those features, one weight vector per operation.
``rank`` orders candidates by predicted time; ``BaseTunner.tune(top_k=...)`` compiles only the first k.

    python -m attention_autotuner_b200.autotuner.cost_model --fit     # refit from logs/*.json, rewrite the weights file
    python -m attention_autotuner_b200.autotuner.cost_model --report  # leave-one-log-out regret of top-k pruning
"""
from __future__ import annotations

import glob
import json
import os
import re

import numpy as np

PKG_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), ".."))
WEIGHTS_PATH = os.path.join(os.path.dirname(__file__), "cost_model_weights.json")
LOG_DIR = os.path.join(PKG_DIR, "logs")

SM_COUNT = 148
CLOCK_GHZ = 1.965                 # boost clock; the fitted weights absorb the clock the logs were taken at
MMA_FLOP_PER_CLK = 8192.0         # dense 16-bit tcgen05 rate of one SM
MUFU_PER_CLK = 16.0               # ex2 per clock and SM


def parse_config_repr(text: str) -> dict:
    """Fields of a ``repr(config)`` line of a tuner log (``Config(...)`` / ``RetBwdConfig(...)``) as a dict."""
    out = {}
    for key, val in re.findall(r"(\w+)=([\w.\-]+)", text):
        if re.fullmatch(r"-?\d+", val):
            out[key] = int(val)
        else:
            out[key] = val
    return out


def _pairs(Lq: int, Lkv: int, causal: bool) -> float:
    """(query, key) pairs that are not masked; causal is bottom-right aligned (key j visible iff j <= i + Lkv - Lq)."""
    if not causal:
        return float(Lq) * Lkv
    return float(np.clip(np.arange(Lq, dtype=np.int64) + (Lkv - Lq) + 1, 0, Lkv).sum())


def blocks(problem: dict) -> float:
    """128 x 128 blocks of (query, key) pairs the launch has to visit, over the whole batch."""
    return problem["B"] * problem["H"] * _pairs(problem["Lq"], problem["Lkv"], problem.get("causal", False)) / (128.0 * 128.0)


FEATURES = {
    "attn": ["tensor", "mufu_1tile", "mufu_2tile", "mufu_2tile_split", "exp_emu", "exp_h2", "handoff_shallow",
             "handoff_deep", "pair", "mma2", "per_cta"],
    "ret": ["tensor", "handoff", "single_cta", "per_item"],
    "ret_bwd": ["tensor", "handoff", "single_cta", "per_item"],
}


def features(op: str, cfg: dict, problem: dict) -> np.ndarray:
    """Feature vector (cycles summed over the launch, in units of 1e6 cycles per SM) of one candidate."""
    nb = blocks(problem) / SM_COUNT / 1e6
    dqk, dv = problem["dqk"], problem["dv"]
    if op == "attn":
        chunk = cfg.get("dv_chunk", min(dv, 256))
        passes = dv / chunk                                          # Q K^T is recomputed once per chunk of V columns
        t_tensor = passes * (128 * 128 * (dqk + chunk) * 2) / MMA_FLOP_PER_CLK
        t_mufu = passes * 128 * 128 / MUFU_PER_CLK
        q_tiles, split = cfg.get("q_tiles", 1), cfg.get("softmax_split", 1)
        emu = cfg.get("exp_emu", 0) / 8.0
        h2 = cfg.get("exp_h2", 0) / 4.0
        stages = cfg.get("kv_stages", 4)
        pair = 1.0 if cfg.get("cta_pair", 0) else 0.0
        tiles = problem["B"] * problem["H"] * np.ceil(problem["Lq"] / 128.0) * passes / SM_COUNT / 1e6
        # the persistent form of the grid has no per-CTA prologue / epilogue to pay; left to the launcher (-1) it is
        # taken up to 40 KV blocks per work item on average (csrc/fa_fwd_launch.cuh)
        persistent = cfg.get("persistent", -1)
        if persistent == -1 and q_tiles == 2 and chunk <= 128 and split == 1 and not cfg.get("exp_emu", 0) \
                and not cfg.get("exp_h2", 0) and cfg.get("mma_warps", 1) == 1 and not cfg.get("cta_pair", 0):
            nblk = np.ceil(problem["Lkv"] / 128.0)
            persistent = 1 if (np.ceil(nblk / 2.0) if problem.get("causal", False) else nblk) <= 40 else 0
        if persistent == 1:
            tiles = 0.0
        return np.array([
            nb * t_tensor,
            nb * t_mufu * (q_tiles == 1),
            nb * t_mufu * (q_tiles == 2 and split == 1),
            nb * t_mufu * (q_tiles == 2 and split == 2),
            nb * t_mufu * emu,
            nb * t_mufu * h2,
            nb * passes * 1000.0 * (stages <= 2),
            nb * passes * 1000.0 * (stages >= 5),
            nb * passes * 1000.0 * pair,
            nb * passes * 1000.0 * (cfg.get("mma_warps", 1) == 2),
            tiles / max(q_tiles, 1) * 10000.0,                       # prologue / epilogue of a CTA
        ])
    # RetNet chain kernels: forward = one launch, backward = three (dV over dv_chunk, dK and dQ over dq_chunk)
    pair = 1.0 if cfg.get("cta_pair", 0) else 0.0
    if op == "ret":
        chunk = cfg.get("dv_chunk", min(dv, 256))
        passes = dv / chunk
        t_tensor = passes * (128 * 128 * (dqk + chunk) * 2) / MMA_FLOP_PER_CLK
        n_pass = passes
        items = problem["B"] * problem["H"] * np.ceil(problem["Lq"] / 128.0) * passes
    else:
        cv, cq = cfg.get("dv_chunk", min(dv, 256)), cfg.get("dq_chunk", min(dqk, 256))
        pv, pq = dv / cv, dqk / cq
        t_tensor = (pv * (dqk + cv) + 2 * pq * (dv + cq)) * 128 * 128 * 2 / MMA_FLOP_PER_CLK
        n_pass = pv + 2 * pq
        items = problem["B"] * problem["H"] * np.ceil(problem["Lq"] / 128.0) * n_pass
    return np.array([
        nb * t_tensor,
        nb * n_pass * 1000.0,
        nb * t_tensor * (1.0 - pair),                                # the single-CTA kernels stream twice the operand bytes
        items / SM_COUNT / 1e6 * 10000.0,
    ])


def cycles_to_ms(mcycles_per_sm: float) -> float:
    return mcycles_per_sm * 1e6 / (CLOCK_GHZ * 1e9) * 1e3


def _problem_of_log(d: dict) -> dict:
    B, H, Lq, dqk = d["shape"]
    return dict(B=B, H=H, Lq=Lq, Lkv=d.get("seqlen_k", Lq), dqk=d["dim_qk"], dv=d["dim_v"],
                causal=bool(d.get("causal", False)) or d["operation"] != "attn")  # the RetNet logs use the decay mask


def load_logs(log_dir: str = LOG_DIR):
    """[(file name, operation, problem, [(config dict, ms), ...])] from every JSON tuner log."""
    out = []
    for path in sorted(glob.glob(os.path.join(log_dir, "profile_result_*.json"))):
        with open(path) as f:
            d = json.load(f)
        rows = [(parse_config_repr(r["config"]), float(r["ms"])) for r in d["results"] if 0 < r["ms"] < 1e7]
        if rows:
            out.append((os.path.basename(path), d["operation"], _problem_of_log(d), rows))
    return out


def fit(logs=None) -> dict:
    """Non-negative least squares of measured ms on the features, per operation. Rows are weighted by 1 / ms so that
    the fast candidates, the ones the ranking has to get right, count as much as the slow ones."""
    from scipy.optimize import nnls
    logs = load_logs() if logs is None else logs
    weights = {}
    for op in FEATURES:
        X, y = [], []
        for _name, lop, problem, rows in logs:
            if lop != op:
                continue
            for cfg, ms in rows:
                X.append(cycles_to_ms(1.0) * features(op, cfg, problem) / ms)
                y.append(1.0)
        if not X:
            continue
        w, _res = nnls(np.array(X), np.array(y))
        weights[op] = {n: float(v) for n, v in zip(FEATURES[op], w)}
    return weights


_weights_cache = None


def load_weights(path: str = WEIGHTS_PATH) -> dict:
    global _weights_cache
    if _weights_cache is None or path != WEIGHTS_PATH:
        with open(path) as f:
            w = json.load(f)
        if path != WEIGHTS_PATH:
            return w
        _weights_cache = w
    return _weights_cache


def predict_ms(op: str, cfg: dict, problem: dict, weights: dict | None = None) -> float:
    w = (weights if weights is not None else load_weights()).get(op)
    if w is None:
        raise KeyError(f"no cost-model weights for operation {op!r}")
    f = features(op, cfg, problem)
    return float(cycles_to_ms(1.0) * sum(w[n] * v for n, v in zip(FEATURES[op], f)))


def rank(op: str, configs: list, problem: dict, weights: dict | None = None) -> list:
    """Candidates sorted by predicted time, fastest first. ``configs`` are config objects (their ``__dict__`` is
    used) or dicts. Ties keep the input order."""
    scored = []
    for i, c in enumerate(configs):
        d = c if isinstance(c, dict) else c.__dict__
        scored.append((predict_ms(op, d, problem, weights), i, c))
    scored.sort(key=lambda t: (t[0], t[1]))
    return [c for _ms, _i, c in scored]


def pruning_report(top_k: int = 5, logs=None) -> list:
    """Leave-one-log-out: fit on every other log, rank the held-out log's candidates, and compare the best measured
    time among the first k with the best of the exhaustive search. Returns one record per log."""
    logs = load_logs() if logs is None else logs
    out = []
    for i, (name, op, problem, rows) in enumerate(logs):
        train = [l for j, l in enumerate(logs) if j != i]
        if not any(l[1] == op for l in train):
            train = logs        # the only log of its operation: in-sample
        w = fit(train)
        order = sorted(range(len(rows)), key=lambda r: predict_ms(op, rows[r][0], problem, w))
        k = min(top_k, len(rows))
        best_all = min(ms for _c, ms in rows)
        best_k = min(rows[r][1] for r in order[:k])
        out.append(dict(log=name, operation=op, candidates=len(rows), top_k=k, best_ms=best_all, best_in_top_k_ms=best_k,
                        regret=best_k / best_all - 1.0,
                        rank_of_best=1 + order.index(min(range(len(rows)), key=lambda r: rows[r][1])),
                        in_sample=train is logs))
    return out


def main():
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--fit", action="store_true", help="refit from the committed logs and rewrite the weights file")
    ap.add_argument("--report", action="store_true")
    ap.add_argument("--top-k", type=int, default=5)
    args = ap.parse_args()
    if args.fit:
        w = fit()
        with open(WEIGHTS_PATH, "w") as f:
            json.dump(w, f, indent=1, sort_keys=True)
        print("wrote", WEIGHTS_PATH)
    if args.report or not args.fit:
        for rec in pruning_report(args.top_k):
            print(json.dumps(rec))


if __name__ == "__main__":
    main()
