"""The engine at the layer sizes of the benchmark model (hidden 4096, 32 query and 8 key/value
heads of 128, feed-forward 12288, vocabulary 151936; one layer, to keep it short): the kernels
the tiny configurations never reach (tcgen05 products and attention, the wide q/k-norm, the
vocabulary product over 151936 rows) under the same ways of cutting the work."""
import json

import pytest


@pytest.mark.gpu
def test_real_layer_sizes_float32_and_bfloat16_alone_and_cut(capsys):
    import bench
    config = dict(bench.CONFIG_8B, num_hidden_layers=1)
    rc = bench.exactness_check(config, seed=8, shape="8b")
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and line["ok"], line
    # true float32 does not depend on how the tokens are cut, to the bit
    assert line["float32_cut_vs_alone_max_abs"] == 0.0
    assert line["bfloat16_cut_vs_float32_max_abs"] <= line["bfloat16_bound"]
    assert line["bfloat16_top1_agrees_with_float32"] >= 0.9


@pytest.mark.gpu
def test_step_logits_last_until_the_next_step_only():
    """What `Engine.step` says of its result: a decode step replayed from a graph writes into
    the buffer of the last replay, so a caller that wants to keep logits copies them."""
    import torch

    import tgo_b200
    from tgo_b200.engine.step import Engine, StepEntry
    from tiny import TINY_A
    model = tgo_b200.open_random(dict(TINY_A), seed=3, dtype="bfloat16").model
    eng = Engine(model, page_size=16, max_tokens=128, num_slots=1)
    eng.admit("a")
    eng.step([StepEntry("a", [1, 2, 3], [2])])
    kept, copies = [], []
    for t in (4, 5, 6, 7, 8, 9):
        out = eng.step([StepEntry("a", [t], [0])])
        kept.append(out)
        copies.append(out.clone())
    # the copies differ from step to step; whatever the kept tensors alias, the last one is
    # the last step's
    assert torch.equal(kept[-1], copies[-1])
    assert not torch.equal(copies[0], copies[-1])
