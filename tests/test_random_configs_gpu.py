"""Seeded random configurations of the architecture, each with a random mix of requests, through
every way of cutting against the plain implementation.  The fixed tiny configurations pin chosen
corners; these draw the corners' neighbours: head sizes in steps of 16 up to 128 (the tensor-core
kernels' 64 and 128 among them), any group size from 1 to 8, widths that are multiples of 8
only, windows shorter and longer than a page on a random subset of the layers, tied and untied
heads, three values of the norms' eps and of theta."""

import numpy as np
import pytest
import torch

import harness

pytestmark = pytest.mark.gpu


def draw_config(seed):
    g = torch.Generator().manual_seed(7000 + seed)

    def pick(options):
        return options[int(torch.randint(0, len(options), (1,), generator=g))]

    n_kv = pick([1, 2, 3, 4])
    group = pick([1, 2, 3, 4, 8])
    head_dim = pick([16, 32, 48, 64, 64, 80, 128, 128])
    layers = pick([1, 2, 3])
    window = pick([None, None, 20, 70, 150])
    types = ["full_attention"] * layers
    if window is not None:
        types = [pick(["full_attention", "sliding_attention"]) for _ in range(layers)]
        if "sliding_attention" not in types:
            types[-1] = "sliding_attention"
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=pick([97, 300, 1000, 2051]),
               hidden_size=8 * pick([5, 9, 12, 16, 20]), intermediate_size=8 * pick([7, 13, 24, 40]),
               num_hidden_layers=layers, num_attention_heads=n_kv * group, num_key_value_heads=n_kv,
               head_dim=head_dim, rms_norm_eps=pick([1e-6, 1e-5, 3e-6]), rope_theta=pick([1e4, 5e5, 5e6]),
               tie_word_embeddings=bool(pick([0, 1])), max_position_embeddings=4096, hidden_act="silu",
               attention_bias=False, rope_scaling=None)
    if window is not None:
        cfg.update(sliding_window=window, use_sliding_window=True, layer_types=types)
    lengths = [int(torch.randint(1, 200, (1,), generator=g)) for _ in range(pick([3, 4, 5]))]
    return cfg, lengths, g


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_random_configuration_in_every_cutting(tmp_path, seed, dtype):
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import write_random_model
    cfg, lengths, g = draw_config(seed)
    stored = torch.float32 if seed % 2 else torch.bfloat16
    folder = write_random_model(str(tmp_path / "model"), config_from_dict(cfg), seed=seed, dtype=stored, gain_std=0.1)
    requests = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    what = f"seed {seed}: {cfg['num_attention_heads']}/{cfg['num_key_value_heads']} heads of {cfg['head_dim']}, " \
           f"window {cfg.get('sliding_window')}, lengths {lengths}"
    whole = harness.replay(folder, dtype, harness.trace_whole(requests), str(tmp_path / "w"))
    harness.check_against_plain(whole, requests, folder, dtype, what + ", whole")
    tail = harness.replay(folder, dtype, harness.trace_tail(requests, 32), str(tmp_path / "t"))
    harness.check_against_plain(tail, requests, folder, dtype, what + ", tail")
    names = list(requests)
    batches = [{k: requests[k] for k in names[:2]}, {k: requests[k] for k in names[2:]}]
    prompt_lens = {k: max(1, len(requests[k]) - (5 + 7 * i) % 40) for i, k in enumerate(names)}
    mixed = harness.replay(folder, dtype, harness.trace_batches(batches, prompt_lens), str(tmp_path / "b"))
    harness.check_against_plain(mixed, requests, folder, dtype, what + ", batches")
    if dtype == "float32":
        for r in requests:
            assert np.array_equal(whole[r], tail[r]) and np.array_equal(whole[r], mixed[r]), \
                f"{what}: float32 logits of {r} depend on the cutting"
