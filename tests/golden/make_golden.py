"""Regenerates tests/golden/mla_golden.json.

Run where the reference tree is mounted (it compiles the reference's own sources through
oracle/Makefile `ref` and executes them):

    python tests/golden/make_golden.py

Attention, YaRN-frequency, KVCache-counter, append and q-RoPE entries are outputs of the REFERENCE's
code.  The append (RMSNorm + NeoX/YaRN RoPE + scatter) and the q RoPE are inline in the reference's forward()
and not callable, so they are reached by running its real from_gguf + forward() on a tiny synthetic deepseek2
GGUF file (tests/golden/tiny_gguf.py) over host stand-ins of the Metal layer (oracle/ref_harness.cpp): the
entries hold what that code read (kv_a, q before rotation) and what it wrote (the cache row, q after rotation).
"append_restated" entries come from the restatement in oracle/mla_oracle.cpp (bf16 storage and very large
positions, which the f16-only reference with its [context_length][576] buffers does not offer); they guard
against regressions only.  Where inputs are not stored, an entry carries the generator arguments and a
SHA-256 of the generated inputs, so a drifting generator is detected instead of silently re-baselined.
"""
import base64
import json
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from mugen_b200 import synth  # noqa: E402
from oracle import binding  # noqa: E402
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import tiny_gguf  # noqa: E402

# A still smaller model whose every decode call is recorded in full (the "block" entries): what the reference's decode
# driver fed into and got out of each layer's attention block, position by position.  The projections inside it run on
# the harness's C++ restatements of the reference's Metal kernels (the shaders cannot run on this host); RMSNorm of
# kv_a, both RoPEs, the attention and the order of the steps are the reference's own host code.
BLOCK_CASE = dict(name="C: block trace, q-LoRA", model=dict(n_heads=2, embed=64, q_lora_rank=32, ffn=32, vocab=8, seed=13,
                                                          context_length=64), positions=10)

# Tiny models driven through the reference's forward(); `steps` = (token, position) calls in order, `keep` =
# the positions whose rows are stored.  The reference writes the row at the caller's position without checking
# that it equals seq_len (src/core/model/transformer.cpp:3982), so model B may jump.
FORWARD_CASES = [
    dict(name="A: q-LoRA, separate k_b/v_b, YaRN factor 40", model=dict(),
         steps=[(p % 16, p) for p in range(67)], keep=[0, 1, 31, 63, 64, 66]),
    dict(name="B: full q, merged kv_b, plain RoPE, eps 1e-5",
         model=dict(q_lora_rank=0, merged_kv_b=True, rope_factor=1.0, eps=1e-5, context_length=8192, seed=11, n_heads=2),
         steps=[(3, 0), (5, 63), (7, 64), (9, 4095), (11, 8191)], keep=[0, 63, 64, 4095, 8191]),
]

ATTN_CASES = [
    # seed, heads, seq_len, w_type, q_scale, exact_in_both
    dict(seed=101, n_heads=2, seq_len=1, w_type=synth.W_F16, q_scale=1.0, exact_in_both=False),
    dict(seed=102, n_heads=3, seq_len=63, w_type=synth.W_F16, q_scale=1.0, exact_in_both=False),
    dict(seed=103, n_heads=4, seq_len=64, w_type=synth.W_F16, q_scale=1.0, exact_in_both=False),
    dict(seed=104, n_heads=4, seq_len=65, w_type=synth.W_F16, q_scale=4.0, exact_in_both=False),
    dict(seed=105, n_heads=16, seq_len=333, w_type=synth.W_F16, q_scale=1.0, exact_in_both=False),
    dict(seed=106, n_heads=4, seq_len=257, w_type=synth.W_Q8_0, q_scale=1.0, exact_in_both=False),
    dict(seed=107, n_heads=4, seq_len=130, w_type=synth.W_Q4_0, q_scale=1.0, exact_in_both=False),
    dict(seed=108, n_heads=8, seq_len=200, w_type=synth.W_F16, q_scale=1.0, exact_in_both=True),
    dict(seed=109, n_heads=8, seq_len=777, w_type=synth.W_F16, q_scale=8.0, exact_in_both=True),
]
YARN_CASES = [
    dict(factor=40.0, orig_ctx=4096, theta=10000.0),    # DeepSeek-V2-Lite
    dict(factor=0.0, orig_ctx=0, theta=10000.0),        # plain RoPE
    dict(factor=1.0, orig_ctx=4096, theta=10000.0),
    dict(factor=40.0, orig_ctx=4096, theta=1000000.0),
    dict(factor=4.0, orig_ctx=32768, theta=50000.0),
]
COUNTER_TRACE = [("advance", 1), ("advance", 1), ("advance", 7), ("truncate", 4), ("advance", 3),
                 ("truncate", 7), ("truncate", 0), ("advance", 5), ("clear", 0), ("advance", 2),
                 ("truncate", 9)]
APPEND_CASES = [
    dict(seed=201, n=5, dt=synth.DT_F16, factor=40.0, orig_ctx=4096, theta=10000.0, eps=1e-6,
         positions=[0, 1, 63, 64, 8191]),
    dict(seed=202, n=4, dt=synth.DT_BF16, factor=40.0, orig_ctx=4096, theta=10000.0, eps=1e-6,
         positions=[0, 5, 16383, 131071]),
    dict(seed=203, n=3, dt=synth.DT_F16, factor=0.0, orig_ctx=0, theta=10000.0, eps=1e-5,
         positions=[2, 100, 4095]),
]


def b64(a: np.ndarray) -> str:
    return base64.b64encode(np.ascontiguousarray(a).tobytes()).decode()


def main() -> None:
    binding.build(ref=True)
    ref = binding.reference()
    assert ref is not None, "reference build missing"
    ora = binding.oracle()
    out = {"attention": [], "yarn": [], "counter": [], "append": []}
    for c in ATTN_CASES:
        case = synth.make_layer_case(c["seed"], c["n_heads"], [c["seq_len"]], synth.DT_F16,
                                     c["w_type"], c["q_scale"], c["exact_in_both"])
        o = ref.attention(case.q[0], case.caches[0], c["seq_len"], case.w_uk, case.w_uv,
                          c["w_type"], c["n_heads"])
        out["attention"].append({**c, "inputs_sha256": case.digest(), "out_f16": b64(o),
                                 "source": "reference cpu_mla_attention"})
    for c in YARN_CASES:
        f = np.array([ref.yarn_rope_freq(i, 64, c["factor"], c["orig_ctx"], c["theta"])
                      for i in range(32)], np.float32)
        out["yarn"].append({**c, "freq_f32": b64(f), "source": "reference yarn_rope_freq"})
    kc = ref.L.ref_kvcache_create(3, 8192)
    lens = []
    for op, n in COUNTER_TRACE:
        if op == "advance":
            ref.L.ref_kvcache_advance(kc, n)
        elif op == "truncate":
            ref.L.ref_kvcache_truncate(kc, n)
        else:
            ref.L.ref_kvcache_clear(kc)
        lens.append(int(ref.L.ref_kvcache_seq_len(kc)))
    ref.L.ref_kvcache_destroy(kc)
    out["counter"].append({"trace": COUNTER_TRACE, "seq_len_after": lens,
                           "source": "reference KVCache (MLA construction)"})
    out["append_restated"] = []
    for c in APPEND_CASES:
        case = synth.make_layer_case(c["seed"], 1, [1] * c["n"], c["dt"])
        rows = ora.append_rows(case.kv_a, c["positions"], case.norm_w, c["eps"], c["factor"],
                               c["orig_ctx"], c["theta"], c["dt"])
        out["append_restated"].append({**c, "inputs_sha256": case.digest(), "rows": b64(rows),
                                       "source": "restatement (oracle/mla_oracle.cpp)"})
    out["q_rope"] = []
    with tempfile.TemporaryDirectory() as tmp:
        for fc in FORWARD_CASES:
            path = os.path.join(tmp, "tiny.gguf")
            tiny_gguf.write(path, tiny_gguf.TinyModel(**fc["model"]))
            mod = ref.load_model(path)
            cfg = mod.cfg
            common = dict(model=fc["name"], factor=cfg["rope_scaling_factor"], orig_ctx=cfg["rope_original_ctx"],
                          theta=cfg["rope_theta"], eps=cfg["rms_norm_eps"], dt=synth.DT_F16)
            norm_w = [mod.weight(L, "kv_a_norm", 1024)[1].view(np.uint16) for L in range(cfg["n_layers"])]
            for token, pos in fc["steps"]:
                taps = mod.forward(token, pos)
                if pos not in fc["keep"]:
                    continue
                for L in range(cfg["n_layers"]):
                    out["append"].append({**common, "layer": L, "position": pos, "kv_a": b64(taps["kv_a_pre"][L]),
                                          "norm_w": b64(norm_w[L]), "row": b64(mod.cache_rows(L, pos, 1)[0]),
                                          "source": "reference forward(), steps G+H"})
                # one layer's q is enough per position (n_heads x 192 values each way)
                out["q_rope"].append({**common, "position": pos, "n_heads": cfg["n_heads"],
                                      "q_in": b64(taps["q_pre"][0]), "q_out": b64(taps["q_post"][0]),
                                      "source": "reference forward(), step E"})
            mod.close()
        path = os.path.join(tmp, "block.gguf")
        tiny_gguf.write(path, tiny_gguf.TinyModel(**BLOCK_CASE["model"]))
        mod = ref.load_model(path)
        out["block"] = {"model": BLOCK_CASE["model"], "name": BLOCK_CASE["name"], "steps": [],
                        "source": "reference forward() on host restatements of its Metal kernels"}
        for pos in range(BLOCK_CASE["positions"]):
            taps = mod.forward(pos % BLOCK_CASE["model"]["vocab"], pos)
            out["block"]["steps"].append({k: b64(v) for k, v in taps.items()})
        mod.close()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mla_golden.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
