"""The whole model at the layer sizes of Qwen3-4B (hidden 2,560, 32 query and 8 kv heads of
128, intermediate 9,728; two layers and a vocabulary of 3,001 keep it to seconds) against the
plain implementation.  The tiny configurations never reach the kernels that serve these sizes
on the product path: the tcgen05 prompt attention, the single-token kernel with the q/k norm
and rotation inside and its cluster merge, the TMA / tcgen05 weight-streaming products for the
o and down projections.  Here they all run inside one model, in every way of cutting."""

import numpy as np
import pytest
import torch

import harness

pytestmark = pytest.mark.gpu

CONFIG = dict(vocab_size=3001, hidden_size=2560, intermediate_size=9728, num_hidden_layers=2,
              num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=5e6,
              tie_word_embeddings=True, max_position_embeddings=4096, architectures=["Qwen3ForCausalLM"])


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import write_random_model
    folder = tmp_path_factory.mktemp("real_sizes") / "model"
    return write_random_model(str(folder), config_from_dict(CONFIG), seed=3, gain_std=0.1)


def requests():
    return {f"r{i}": torch.randint(0, CONFIG["vocab_size"], (n,), generator=torch.Generator().manual_seed(50 + i)).tolist()
            for i, n in enumerate([200, 70, 131])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_in_every_cutting(model_dir, tmp_path, dtype):
    from thing_htn_2026_b200 import ops
    reqs = requests()
    before = ops.launch_count
    whole = harness.replay(model_dir, dtype, harness.trace_whole(reqs), str(tmp_path / "w"))
    harness.check_against_plain(whole, reqs, model_dir, dtype, "whole")
    tail = harness.replay(model_dir, dtype, harness.trace_tail(reqs, 32), str(tmp_path / "t"))
    harness.check_against_plain(tail, reqs, model_dir, dtype, "tail")
    batches = [{k: reqs[k] for k in ("r0", "r1")}, {"r2": reqs["r2"]}]
    mixed = harness.replay(model_dir, dtype, harness.trace_batches(batches, {"r0": 150, "r1": 64, "r2": 1}),
                           str(tmp_path / "b"))
    harness.check_against_plain(mixed, reqs, model_dir, dtype, "batches")
    assert ops.launch_count > before
    if dtype == "float32":
        for r in reqs:
            assert np.array_equal(whole[r], tail[r]) and np.array_equal(whole[r], mixed[r]), \
                f"{r}: float32 logits depend on the cutting"
