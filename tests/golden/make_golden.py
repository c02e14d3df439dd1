"""Generate the golden fixtures under tests/golden/ from the reference tree.

Run where the reference checkout is present (REFERENCE=<its path>, or a directory "reference" beside this repository):
    python tests/golden/make_golden.py

Writes
  layer0.npz            input/output activation pairs of every in-scope op of Qwen3-0.6B
                        layer 0, as exported by the reference from HF Transformers fp32
                        (artifacts/phase1/qwen3_layer0/*.f32; large projection weights are
                        left out, they are not needed: each op's input AND output is on disk)
  logits_last_rows.npz  the last logits row of the two full-prefill cases with the greedy id
                        and top-5 ids the reference recorded for them
                        (artifacts/phase25/qwen3_full_prefill/case_seq{4,8})
  c1_reference.npz      outputs of the reference's own compiled CPU operators (oracle/_ref) on
                        the seeded configuration-1 inputs (cuda_llm_b200.workloads.config1)
  small_reference.npz   the same for small fp16 cases of configurations 2, 3 and 5 and of the
                        decode-size LM head (inputs regenerated from their seeds by the tests)
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

REFERENCE = oracle.reference_tree()   # $REFERENCE, else a directory named "reference" beside this repository
if REFERENCE is None:
    raise SystemExit("make_golden.py: set REFERENCE to the root of the reference's source tree")
from cuda_llm_b200 import workloads as wl  # noqa: E402


def layer0():
    d = os.path.join(REFERENCE, "artifacts/phase1/qwen3_layer0")
    keep = ["input_layernorm_weight", "q_norm_weight", "k_norm_weight", "post_attention_layernorm_weight",
            "hidden_states", "input_norm", "q_linear", "q_norm_output", "k_linear", "k_norm_output", "q_rope", "k_rope",
            "o_proj_output", "attention_residual", "post_attention_norm", "gate_proj_output", "up_proj_output",
            "swiglu_output", "down_proj_output", "layer_output", "position_ids"]
    out = {}
    for line in open(os.path.join(d, "manifest.txt")):
        name, fname, rank, *dims = line.split()
        if name in keep:
            out[name] = np.fromfile(os.path.join(d, fname), dtype="<f4").reshape([int(x) for x in dims])
    cfg = dict(l.split(None, 1) for l in open(os.path.join(d, "config.txt")))
    out["rms_norm_eps"] = np.float32(cfg["rms_norm_eps"])
    out["rope_theta"] = np.float32(cfg["rope_theta"])
    np.savez_compressed(os.path.join(HERE, "layer0.npz"), **out)


def logits():
    out = {}
    for case in ("case_seq4", "case_seq8"):
        d = os.path.join(REFERENCE, "artifacts/phase25/qwen3_full_prefill", case)
        rows = np.fromfile(os.path.join(d, "logits.f32.bin"), dtype="<f4").reshape(-1, wl.VOCAB)
        out[case + "_last_row"] = rows[-1].copy()
        out[case + "_greedy_id"] = np.fromfile(os.path.join(d, "last_token_greedy_id.i32.bin"), dtype="<i4")
        out[case + "_top5_ids"] = np.fromfile(os.path.join(d, "last_token_top5_ids.i32.bin"), dtype="<i4")
        out[case + "_top5_logits"] = np.fromfile(os.path.join(d, "last_token_top5_logits.f32.bin"), dtype="<f4")
    np.savez_compressed(os.path.join(HERE, "logits_last_rows.npz"), **out)


def reference_outputs():
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("oracle/_ref is not built: run `make -C oracle ref` where the reference tree exists")
    c = wl.config1()
    res, nrm = ref.add_rms_norm(c["x"], c["res"], c["gamma"], wl.EPS)
    qn = ref.rms_norm(c["q"].reshape(-1, 128), c["gamma_q"], wl.EPS).reshape(c["q"].shape)
    kn = ref.rms_norm(c["k"].reshape(-1, 128), c["gamma_k"], wl.EPS).reshape(c["k"].shape)
    np.savez_compressed(
        os.path.join(HERE, "c1_reference.npz"), residual=res, normalized=nrm, q_norm=qn, k_norm=kn,
        q_rope=ref.rope(qn, c["positions"], wl.THETA), k_rope=ref.rope(kn, c["positions"], wl.THETA),
        swiglu=ref.swiglu(c["gate"], c["up"]), gather=ref.embedding_lookup(c["table"], c["ids"]),
        ids=c["ids"])

    port = oracle.port()
    small = {}
    c2 = wl.config2(64, 1024)                       # fp16 inputs, de-quantised exactly for the F32-only CPU ops
    f = {k: port.decode_f16(v.view(np.uint16)) for k, v in c2.items()}
    small["c2_residual"], small["c2_normalized"] = ref.add_rms_norm(f["x"], f["res"], f["gamma"], wl.EPS)
    c3 = wl.config3(tokens=64)
    q, k = port.decode_f16(c3["q"].view(np.uint16)), port.decode_f16(c3["k"].view(np.uint16))
    gq, gk = port.decode_f16(c3["gamma_q"].view(np.uint16)), port.decode_f16(c3["gamma_k"].view(np.uint16))
    small["c3_q"] = ref.rope(ref.rms_norm(q.reshape(-1, 128), gq, wl.EPS).reshape(q.shape), c3["positions"], wl.THETA)
    small["c3_k"] = ref.rope(ref.rms_norm(k.reshape(-1, 128), gk, wl.EPS).reshape(k.shape), c3["positions"], wl.THETA)
    c5 = wl.config5(rows=4, vocab=8192, seed=5002)
    small["c5_softmax"] = ref.softmax(c5["logits"])
    lm = wl.lm_head_case(rows=4, hidden=1024, vocab=640, seed=6002, dtype=np.float16)
    small["lm_head_logits"] = ref.lm_head(port.decode_f16(lm["hidden"].view(np.uint16)),
                                          port.decode_f16(lm["table"].view(np.uint16)))
    np.savez_compressed(os.path.join(HERE, "small_reference.npz"), **small)


if __name__ == "__main__":
    layer0()
    logits()
    reference_outputs()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
