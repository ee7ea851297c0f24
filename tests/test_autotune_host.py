"""Host logic of the autotuner: which configuration enters the tuning table, and the round trip of
timing rows through a CSV file into the latency models (no GPU involved)."""

import csv
import math

from spio_b200.kernels import autotune
from spio_b200.kernels.conv2d_gw8_kernel import Conv2dGw8Config
from spio_b200.kernels.conv2d_gw8_params import Conv2dGw8Params


def test_a_table_entry_must_beat_the_planners_defaults_by_a_margin():
    default = Conv2dGw8Config()
    a = Conv2dGw8Config(wpg=2, tpw=4, pps=2, ns=3)
    b = Conv2dGw8Config(wpg=1, tpw=8, pps=1)
    # 2 % faster than the defaults: within the noise, the defaults stay
    ms, cfg = autotune.pick([(0.0980, a), (0.1000, default), (0.1500, b)])
    assert cfg == default and ms == 0.1000
    # 5 % faster: the configuration is taken
    ms, cfg = autotune.pick([(0.0950, a), (0.1000, default), (0.1500, b)])
    assert cfg == a and ms == 0.0950
    # the defaults are the fastest
    ms, cfg = autotune.pick([(0.1000, default), (0.1010, a)])
    assert cfg == default
    # no default among the candidates (an explicit list of configurations): plain minimum
    ms, cfg = autotune.pick([(0.0990, a), (0.1500, b)])
    assert cfg == a
    assert 0.9 < autotune.TABLE_MARGIN < 1.0


def test_rows_round_trip_and_models_fit(tmp_path):
    params = Conv2dGw8Params(n=64, c=64, h=28, w=28, padding=1, r=3, s=3)
    rows = []
    for wpg in (1, 2):
        for tpw in (2, 4, 8):
            for pps in (1, 2):
                cfg = Conv2dGw8Config(wpg=wpg, tpw=tpw, pps=pps)
                ms = 0.02 + 0.004 * wpg + 0.001 * tpw + 0.003 * pps   # a made-up but learnable latency
                rows.append(dict(autotune.feature_row("spio_conv2d_gw8_fprop", params, cfg, ms),
                                 kernel="spio_conv2d_gw8_fprop"))
    rows = rows * 3
    path = tmp_path / "rows.csv"
    fields = ["kernel"] + sorted({k for r in rows for k in r if k != "kernel"})
    with path.open("w", newline="") as fh:
        wr = csv.DictWriter(fh, fieldnames=fields, restval=0)
        wr.writeheader()
        wr.writerows(rows)
    back = autotune.read_rows(path)
    assert list(back) == ["spio_conv2d_gw8_fprop"] and len(back["spio_conv2d_gw8_fprop"]) == len(rows)
    autotune.fit_models(back, tmp_path)
    import json

    from spio_b200.kernels.gbt_model import GbtModel

    model = GbtModel.from_json(json.loads((tmp_path / "model__spio_conv2d_gw8_fprop__sm_100a.json").read_text()))
    feats = [{k: v for k, v in r.items() if k != "ms"} for r in back["spio_conv2d_gw8_fprop"]]
    pred = model.predict(feats)
    want = [math.log(r["ms"]) for r in back["spio_conv2d_gw8_fprop"]]
    assert max(abs(p - w) for p, w in zip(pred, want)) < 0.05
    # the model ranks the fastest configuration first
    assert min(range(len(pred)), key=lambda i: pred[i]) == min(range(len(want)), key=lambda i: want[i])
