"""Skip-softmax deployment resolution and per-sequence thresholds (host side)."""
import math

import pytest
import torch

from tensorrt_edge_llm_b200 import skip_softmax as ss
from tensorrt_edge_llm_b200.config import ModelConfig


def test_table_validation_and_lookup():
    t = ss.validate_table([[8192, 300], [0, 50], [32768, 900]])
    assert t == [[0, 50], [8192, 300], [32768, 900]]
    assert ss.scale_for_length(t, 100) == 50 and ss.scale_for_length(t, 8192) == 300 and ss.scale_for_length(t, 40000) == 900
    assert ss.scale_for_length([[4096, 200]], 1000) is None                    # below the first calibrated length: dense
    for bad in ([], [[1, 2, 3]], [[-1, 5]], [[1.5, 2]], [[4, 5], [4, 6]], "x", [[True, 1]]):
        with pytest.raises(ss.SkipSoftmaxConfigError):
            ss.validate_table(bad)
    with pytest.raises(ss.SkipSoftmaxConfigError):
        ss.validate_table([[i, 1] for i in range(200)])


def test_resolution_order():
    root = {"skip_softmax_prefill_scale_table": [[0, 100]], "skip_softmax_prefill_scale_tables": {"75%": [[0, 700]], "50%": [[0, 300]]},
            "skip_softmax_prefill_calibration": {"a": 10.0, "b": 4.0}, "skip_softmax_decode_scale_table": [[4096, 80]]}
    d = ss.resolve(root)
    assert d.prefill_table == [[0, 100]] and d.decode_table == [[4096, 80]] and d.enabled
    assert ss.resolve(root, prefill_table=[]).prefill_table is None                           # explicit dense flag
    assert ss.resolve(root, prefill_table=[[0, 9]]).prefill_table == [[0, 9]]                 # explicit table flag
    assert ss.resolve(root, prefill_target_sparsity=0.75).prefill_table == [[0, 700]]         # tier of the flag's target
    d = ss.resolve(root, prefill_target_sparsity=0.6)                                         # no tier: the {a, b} fit
    assert d.prefill_table == [[0, round(10.0 * math.exp(4.0 * 0.6))]] and d.prefill_target_sparsity == 0.6
    assert ss.resolve(dict(root, skip_softmax_prefill_target_sparsity=0.5)).prefill_table == [[0, 300]]    # checkpoint tier beats its plain table
    assert ss.resolve(root, decode_table=[]).decode_table is None and ss.resolve(root, decode_table=[]).prefill_table == [[0, 100]]
    with pytest.raises(ss.SkipSoftmaxConfigError):
        ss.resolve({}, prefill_target_sparsity=0.5)                                           # a target with nothing to derive S from
    with pytest.raises(ss.SkipSoftmaxConfigError):
        ss.resolve({}, decode_target_sparsity=1.5)
    # the text config is read before the checkpoint root
    assert ss.resolve(root, {"skip_softmax_prefill_scale_table": [[0, 7]]}).prefill_table == [[0, 7]]
    assert not ss.resolve({}).enabled


def test_thresholds_per_sequence_and_config_parsing():
    table = [[2048, 64]]
    thr = ss.thresholds_log2(table, [100, 2048, 8192])
    assert thr[0] == float("-inf") and torch.allclose(thr[1:], torch.tensor([math.log2(64 / 2048), math.log2(64 / 8192)]))
    assert ss.thresholds_log2(table, [10, 20]) is None and ss.thresholds_log2(None, [5000]) is None
    assert ss.thresholds_log2([[0, 500]], [100]) is None                                      # S >= L: lambda >= 1 is meaningless, dense
    hf = dict(model_type="llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, skip_softmax_prefill_scale_table=[[1024, 40]])
    cfg = ModelConfig.from_hf_dict(hf)
    assert cfg.skip_softmax_prefill_table == [[1024, 40]] and cfg.skip_softmax_decode_table is None
    assert ModelConfig.from_dict(cfg.to_dict()).skip_softmax_prefill_table == [[1024, 40]]
