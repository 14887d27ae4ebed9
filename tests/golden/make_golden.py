"""Makes tests/golden/reference_outputs.json by running the REFERENCE's own CPU code on a
tiny random model: its torch twins (engine/kernels/torch_ref.py) through its own step
functions (engine/engine.py ``_prefill_slice`` and ``_step``), in float32 and in bfloat16.

    python tests/golden/make_golden.py /path/to/reference

The reference's constructor loads weights through a library loader, which is not used
here: the Engine object is made without calling ``__init__`` and is given the attributes
its step functions read (the weights of tests/golden/common.py, fused as
engine/engine.py:214-222 fuses them).  For float32 the weights, caches and rotary tables
are float32 (the reference's formulas are dtype-generic; its tables are rounded to
bfloat16 only because its checkpoints are).  The LM-head logits, which the reference never
returns, are caught by wrapping ``F.linear`` where the head is applied.
"""

import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import common  # noqa: E402


def build_engine(reference_root, dtype):
    os.environ.setdefault("TRITON_CACHE_DIR", tempfile.mkdtemp())
    os.environ["DRYFT_ENGINE_DEVICE"] = "cpu"
    os.environ["DRYFT_ENGINE_TRITON"] = "0"
    sys.path.insert(0, os.path.join(reference_root, "engine"))
    import engine as ref
    ref.CONFIG["log"] = False
    c = common.CONFIG
    w = {k: v.to(dtype) for k, v in common.weights().items()}
    eng = object.__new__(ref.Engine)
    eng.device, eng.is_cuda, eng.use_triton, eng.use_graphs = torch.device("cpu"), False, False, False
    eng.H, eng.I, eng.V, eng.L = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["num_hidden_layers"]
    eng.Nq, eng.Nkv, eng.D = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    eng.eps, eng.theta, eng.scale = c["rms_norm_eps"], c["rope_theta"], c["head_dim"] ** -0.5
    eng.layers = []
    for i in range(eng.L):
        p = f"model.layers.{i}."
        layer = ref._Layer()
        layer.ln1 = w[p + "input_layernorm.weight"]
        layer.w_qkv = torch.cat([w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                                 w[p + "self_attn.v_proj.weight"]], dim=0).contiguous()
        layer.q_norm, layer.k_norm = w[p + "self_attn.q_norm.weight"], w[p + "self_attn.k_norm.weight"]
        layer.w_o = w[p + "self_attn.o_proj.weight"]
        layer.ln2 = w[p + "post_attention_layernorm.weight"]
        layer.w_gu = torch.cat([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]], dim=0).contiguous()
        layer.w_down = w[p + "mlp.down_proj.weight"]
        eng.layers.append(layer)
    eng.embed = w["model.embed_tokens.weight"]
    eng.lm_head = eng.embed
    eng.final_norm = w["model.norm.weight"]
    eng.graphs, eng.use_fused, eng.w_t = {}, {}, {}
    eng.layout_t = {"decode": set(), "prefill": set()}
    eng.sdpa_gqa, eng.num_splits, eng.diag = None, 1, []
    eng._rope_max = 0
    eng._ensure_rope(1024)
    if dtype == torch.float32:      # the same table formula (engine/engine.py:238-247), not rounded
        inv_freq = 1.0 / (eng.theta ** (torch.arange(0, eng.D, 2, dtype=torch.int64).float() / eng.D))
        freqs = torch.arange(eng.cos_tab.shape[0], dtype=torch.float32)[:, None] * inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        eng.cos_tab, eng.sin_tab = emb.cos().contiguous(), emb.sin().contiguous()
    eng._select_ops()
    cap = 64
    shape = (common.BATCH, eng.Nkv, cap, eng.D)
    eng.k_cache = [torch.zeros(shape, dtype=dtype) for _ in range(eng.L)]
    eng.v_cache = [torch.zeros(shape, dtype=dtype) for _ in range(eng.L)]
    eng.B, eng.CAP = common.BATCH, cap
    return ref, eng


def run(reference_root, dtype):
    ref, eng = build_engine(reference_root, dtype)
    caught = []
    plain_linear = ref.F.linear

    def spy(x, weight, bias=None):
        out = plain_linear(x, weight, bias)
        if weight is eng.lm_head and x.shape[-1] == eng.H:
            caught.append(out.float().clone())
        return out

    ref.F.linear = spy
    try:
        with torch.inference_mode():
            ids = common.prompts()
            first = eng._prefill_slice(ids, 0)
            tokens = [first.tolist()]
            pos = torch.full((common.BATCH,), common.PROMPT, dtype=torch.int32)
            current = first
            for _ in range(common.STEPS - 1):
                current = eng._step(current.view(-1, 1), pos, 1)
                pos += 1
                tokens.append(current.tolist())
    finally:
        ref.F.linear = plain_linear
    assert len(caught) == common.STEPS, len(caught)
    logits = torch.stack(caught, dim=1)               # [B, STEPS, V]: the rows that chose each token
    return {"tokens": tokens, "logits": logits.tolist()}


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py REFERENCE_CHECKOUT")
    root = sys.argv[1]
    out = {"float32": run(root, torch.float32)}
    # a fresh import state is not needed: the module keeps no weights
    out["bfloat16"] = run(root, torch.bfloat16)
    out["note"] = ("logits[b][n] are the reference's LM-head outputs that chose generated token n of sequence b "
                   "(bfloat16 run: its logits are bfloat16 values)")
    with open(os.path.join(HERE, "reference_outputs.json"), "w") as handle:
        json.dump(out, handle)
    print("wrote reference_outputs.json", {k: len(v["tokens"]) for k, v in out.items() if k != "note"})


if __name__ == "__main__":
    main()
