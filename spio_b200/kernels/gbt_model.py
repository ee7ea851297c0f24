"""Gradient-boosted regression trees kept as plain JSON and evaluated in pure Python.

The reference predicts kernel latency with XGBoost boosters fetched at run time
(spio/kernels/performance_model_cache.py:226-249); this package ships its models as JSON
next to the code, so prediction needs neither xgboost nor a network.  ``fit`` is a small
least-squares boosting implementation (exact greedy splits) adequate for the few thousand
timing rows an autotuning sweep produces.
"""

from __future__ import annotations

from typing import Dict, List, Sequence


class GbtModel:
    def __init__(self, features: List[str], base: float, rate: float, trees: List[list],
                 ranges: Dict[str, List[float]] = None):
        self.features = features
        # [min, max] of every feature in the training rows; predictions outside are guesses
        self.ranges = ranges or {}
        self.base = base
        self.rate = rate
        # tree = list of nodes; node = [feature_index, threshold, left, right] or [-1, value]
        self.trees = trees

    # ------------------------------------------------------------ prediction
    def _row(self, row: Dict[str, float]) -> List[float]:
        return [float(row.get(f, 0.0)) for f in self.features]

    def predict(self, rows: Sequence[Dict[str, float]]) -> List[float]:
        out = []
        for row in rows:
            x = self._row(row)
            y = self.base
            for tree in self.trees:
                node = tree[0]
                while node[0] >= 0:
                    node = tree[node[2] if x[node[0]] <= node[1] else node[3]]
                y += self.rate * node[1]
            out.append(y)
        return out

    # ------------------------------------------------------------ (de)serialisation
    def covers(self, row: Dict[str, float], names: Sequence[str]) -> bool:
        """True when the named features of ``row`` lie inside the training ranges."""
        for name in names:
            lo_hi = self.ranges.get(name)
            if lo_hi is None or not lo_hi[0] <= float(row.get(name, 0.0)) <= lo_hi[1]:
                return False
        return True

    def to_json(self) -> dict:
        return {"features": self.features, "base": self.base, "rate": self.rate, "trees": self.trees,
                "ranges": self.ranges}

    @classmethod
    def from_json(cls, obj: dict) -> "GbtModel":
        return cls(list(obj["features"]), float(obj["base"]), float(obj["rate"]), obj["trees"],
                   obj.get("ranges"))

    # ------------------------------------------------------------ training
    @classmethod
    def fit(cls, rows: Sequence[Dict[str, float]], target: Sequence[float], n_trees: int = 200,
            depth: int = 4, learning_rate: float = 0.1, min_leaf: int = 1) -> "GbtModel":
        features = sorted({k for r in rows for k in r})
        xs = [[float(r.get(f, 0.0)) for f in features] for r in rows]
        ys = [float(t) for t in target]
        base = sum(ys) / len(ys)
        resid = [y - base for y in ys]
        trees = []
        for _ in range(n_trees):
            tree: List[list] = []
            _grow(tree, xs, resid, list(range(len(xs))), depth, min_leaf)
            trees.append(tree)
            for i, x in enumerate(xs):
                node = tree[0]
                while node[0] >= 0:
                    node = tree[node[2] if x[node[0]] <= node[1] else node[3]]
                resid[i] -= learning_rate * node[1]
        ranges = {f: [min(x[i] for x in xs), max(x[i] for x in xs)] for i, f in enumerate(features)}
        return cls(features, base, learning_rate, trees, ranges)


def _grow(tree: List[list], xs, resid, idx: List[int], depth: int, min_leaf: int) -> int:
    """Append the subtree for samples ``idx`` and return the index of its root node."""
    me = len(tree)
    tree.append(None)
    total = sum(resid[i] for i in idx)
    mean = total / len(idx)
    best = None
    if depth > 0 and len(idx) >= 2 * min_leaf:
        for f in range(len(xs[0])):
            order = sorted(idx, key=lambda i: xs[i][f])
            left_sum = 0.0
            for pos in range(1, len(order)):
                left_sum += resid[order[pos - 1]]
                if xs[order[pos]][f] == xs[order[pos - 1]][f]:
                    continue
                if pos < min_leaf or len(order) - pos < min_leaf:
                    continue
                right_sum = total - left_sum
                gain = left_sum * left_sum / pos + right_sum * right_sum / (len(order) - pos)
                if best is None or gain > best[0]:
                    thr = 0.5 * (xs[order[pos]][f] + xs[order[pos - 1]][f])
                    best = (gain, f, thr, order[:pos], order[pos:])
    if best is None or best[0] <= total * total / len(idx) + 1e-12:
        tree[me] = [-1, mean]
        return me
    _, f, thr, left, right = best
    li = _grow(tree, xs, resid, left, depth - 1, min_leaf)
    ri = _grow(tree, xs, resid, right, depth - 1, min_leaf)
    tree[me] = [f, thr, li, ri]
    return me
