"""The step time line: stamps between the kernels of a step, eager and inside a captured graph."""
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


def test_time_line_of_a_step(model_folders):
    from boring_llm_b200.config import EngineOptions
    from boring_llm_b200.engine.runner import ModelRunner, StepEntry
    from boring_llm_b200.kernels import ops
    from boring_llm_b200.models import load_model
    d = model_folders("A", "bfloat16", 0.02)
    cfg, model = load_model(d, "bfloat16", "cuda:0")
    runner = ModelRunner(model, EngineOptions(dtype="bfloat16", max_tokens=256, ctx_size=128, max_num_seqs=4))
    runner.step([StepEntry("a", helpers.random_tokens(256, 20, 1), [19])])
    with ops.StepTrace("cuda:0") as tr:
        runner.step([StepEntry("b", helpers.random_tokens(256, 70, 2), [69])])       # a portion: kernels launched one by one
    d1 = tr.durations()
    names = [n for n, _ in d1]
    assert names[0] == "bl_embed" and "bl_attention_prefill" in names and names.count("bl_gemm_tc") >= 2 * cfg.num_hidden_layers
    assert all(0 < us < 1e5 for _, us in d1)
    before = ops.launch_count
    with ops.StepTrace("cuda:0") as tr2:
        runner.step([StepEntry("a", [5], [0]), StepEntry("b", [6], [0])])          # decode: captured, stamps inside the graph
    assert runner.graph_steps == 1
    d2 = tr2.durations()
    assert "bl_norm_qkv_rope" in [n for n, _ in d2] and "bl_attention_decode" in [n for n, _ in d2]
    assert ops._trace is None and ops.launch_count > before
