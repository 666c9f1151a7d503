"""Host-side planning of the prefill fast paths (which runs of a step's rows take them): pure index logic, no device."""
import types

import numpy as np

from plow_b200.runtime.engine import TokenBatch


def _batch(runs):
    """runs: [(slot, first position, rows)] laid out back to back."""
    seq = np.concatenate([np.full(n, s, np.int32) for s, _, n in runs])
    pos = np.concatenate([np.arange(p, p + n, dtype=np.int32) for _, p, n in runs])
    return TokenBatch(np.zeros(len(seq), np.int32), pos, seq, np.array([len(seq) - 1], np.int32))


def test_gdn_chunked_plan_splits_long_runs_from_the_rest():
    from plow_b200.runtime.gpu_engine import GpuEngine
    plan = GpuEngine._plan_gdn_prefill
    me = types.SimpleNamespace(GDN_CHUNKED_MIN_RUN=128)
    # a continuing long run, a fresh short one, then the program's padding rows
    p = plan(me, _batch([(0, 200, 200), (1, 0, 37)]), 256)
    assert p["chunked"] == [(0, 0, 200, False)] and p["rest"] == [(200, 256)] and p["R"] == 256
    # two long runs, the second fresh; a short run between them; no padding
    p = plan(me, _batch([(3, 64, 130), (2, 5, 10), (1, 0, 300)]), 440)
    assert p["chunked"] == [(3, 0, 130, False), (1, 140, 440, True)] and p["rest"] == [(130, 140)]
    # nothing long enough, or the feature off: no plan
    assert plan(me, _batch([(0, 0, 100), (1, 0, 27)]), 128) is None
    assert plan(types.SimpleNamespace(GDN_CHUNKED_MIN_RUN=0), _batch([(0, 0, 400)]), 512) is None
    # a position gap inside one slot's rows starts a new run (never merged into one chunked span)
    p = plan(me, _batch([(0, 0, 150), (0, 500, 150)]), 300)
    assert p["chunked"] == [(0, 0, 150, True)] and p["rest"] == [(150, 300)]


def test_mla_materialised_plan_masks_riders_and_respects_the_budget():
    import torch
    from plow_b200.runtime.gpu_engine import GpuEngine
    plan = GpuEngine._plan_mla_prefill

    def me(budget=16384, rows=512):
        return types.SimpleNamespace(MLA_PREFILL_MIN_RUN=64, MLA_PREFILL_BUDGET=budget, max_ctx=8192,
                                     h_plan=torch.zeros(2 * rows + 4 * 8, dtype=torch.int32), d_plan=torch.zeros(2 * rows + 4 * 8, dtype=torch.int32))
    # a prefilling run after a cached prefix, a decode rider, a second prefilling run; 12 padding rows
    m = me()
    b = _batch([(2, 100, 200), (5, 900, 1), (1, 0, 299)])
    p = plan(m, b, 512)
    assert p["n_spans"] == 2 and p["riders"] and p["R"] == 512
    spans = p["spans"].view(-1, 4).tolist()
    assert spans == [[2, 300, 0, 0], [1, 299, 320, 0]]                 # (slot, cached tokens, base rounded to 64, -)
    assert p["total"] == 320 + 320 and p["max_tiles"] == 5
    pos, kv = p["pos"].tolist(), p["kvlen"].tolist()
    assert pos[:200] == list(range(100, 300)) and pos[200] == -1 and pos[201:500] == list(range(299)) and set(pos[500:]) == {-1}
    assert set(kv[:200]) == {0} and kv[200] == 901 and set(kv[201:500]) == {0} and set(kv[500:]) == {0}
    # the budget keeps a second request on the absorbed kernels when its K / V would not fit
    p = plan(me(budget=512), _batch([(2, 100, 200), (1, 0, 299)]), 512)
    assert p["n_spans"] == 1 and p["riders"] and p["kvlen"].tolist()[200:499] == list(range(1, 300))
    # short runs only: no plan
    assert plan(me(), _batch([(0, 0, 40), (1, 7, 30)]), 128) is None
