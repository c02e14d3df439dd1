"""The `*_out` operators allocate nothing, never synchronise and copy nothing to the host, so a
decoder layer's operator sequence can be recorded into a CUDA graph and replayed, as the reference
does for its decode step (src/qwen3_cuda_model.cpp:797-816).  The GEMMs and attention between the
operators are outside this library; their outputs are stand-in tensors here."""
import numpy as np
import pytest
import torch

from cuda_llm_b200 import ops, workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer_ops(t, bufs):
    """The in-scope operators of one Qwen3 decoder layer step, in the reference's order
    (src/qwen3_layer_cuda.cu:285-325), followed by the final norm and a row argmax."""
    ops.cuda_rms_norm_out(t["hidden"], t["w_in"], wl.EPS, bufs["normed"])
    ops.qk_norm_rope_out(t["q"], t["k"], t["w_q"], t["w_k"], t["pos"], wl.EPS, wl.THETA, bufs["q"], bufs["k"])
    ops.cuda_add_rms_norm_out(t["hidden"], t["o_proj"], t["w_post"], wl.EPS, bufs["residual"], bufs["post"])
    ops.cuda_swiglu_out(t["gate"], t["up"], bufs["act"])
    ops.cuda_add_out(bufs["residual"], t["down"], bufs["out"])
    ops.cuda_rms_norm_out(bufs["out"], t["w_in"], wl.EPS, bufs["final"])
    ops.argmax_rows_out(t["logits"], bufs["ids"])


@pytest.mark.parametrize("batch", [1, 4])
def test_layer_operator_sequence_replays_from_a_cuda_graph(b2, batch):
    rng = np.random.default_rng(batch)
    h = lambda *s: torch.from_numpy(wl.normal(rng, s, dtype=np.float16)).to(DEV)
    g = lambda n: torch.from_numpy(wl.gamma(rng, n, dtype=np.float16)).to(DEV)
    t = {"hidden": h(batch, 1024), "o_proj": h(batch, 1024), "down": h(batch, 1024), "q": h(batch, 16, 128),
         "k": h(batch, 8, 128), "gate": h(batch, 3072), "up": h(batch, 3072), "w_in": g(1024), "w_post": g(1024),
         "w_q": g(128), "w_k": g(128), "pos": torch.arange(7, 7 + batch, dtype=torch.int32, device=DEV),
         "logits": torch.from_numpy(wl.normal(rng, (batch, wl.VOCAB), 4.0)).to(DEV)}

    def fresh():
        e = lambda *s: torch.zeros(*s, dtype=torch.float16, device=DEV)
        return {"normed": e(batch, 1024), "q": e(batch, 16, 128), "k": e(batch, 8, 128), "residual": e(batch, 1024),
                "post": e(batch, 1024), "act": e(batch, 3072), "out": e(batch, 1024), "final": e(batch, 1024),
                "ids": torch.zeros(batch, dtype=torch.int32, device=DEV)}

    eager = fresh()
    _layer_ops(t, eager)                       # also warms the library's per-device state before capture
    torch.cuda.synchronize()

    captured = fresh()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            _layer_ops(t, captured)
    for name, buf in captured.items():         # nothing ran during capture
        assert int(buf.abs().sum().item()) == 0 or name == "ids"
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for name in eager:
        assert torch.equal(eager[name], captured[name]), name
    # new inputs, same graph: the replay reads the tensors in place
    t["hidden"].copy_(h(batch, 1024))
    t["logits"][:, 5] = 1e4
    graph.replay()
    again = fresh()
    _layer_ops(t, again)
    torch.cuda.synchronize()
    for name in again:
        assert torch.equal(again[name], captured[name]), name
    assert captured["ids"].tolist() == [5] * batch


def test_sampling_and_the_paged_attention_prologue_replay_from_a_cuda_graph(b2):
    """b2_sample_rows (a memset and kernels only) and b2_qk_norm_rope_paged are capturable like the rest: the graph
    replays the draw and the cache writes on whatever the input tensors hold at replay time."""
    from cuda_llm_b200.ops import SamplingConfig
    rng = np.random.default_rng(11)
    batch, heads, kv_heads, dim, block_size = 4, 16, 8, 128, 16
    h = lambda *s: torch.from_numpy(wl.normal(rng, s, dtype=np.float16)).to(DEV)
    logits = torch.from_numpy(wl.normal(rng, (batch, wl.VOCAB), 4.0)).to(DEV)
    offsets = torch.arange(batch, dtype=torch.int64, device=DEV)
    cfg = SamplingConfig(temperature=0.8, top_k=50, top_p=0.95, seed=3)
    q, k, v = h(batch, heads, dim), h(batch, kv_heads, dim), h(batch, kv_heads, dim)
    gq, gk = torch.from_numpy(wl.gamma(rng, dim, dtype=np.float16)).to(DEV), torch.from_numpy(wl.gamma(rng, dim, dtype=np.float16)).to(DEV)
    pos = torch.tensor([5, 17, 0, 31], dtype=torch.int32, device=DEV)
    tables = torch.arange(batch * 2, dtype=torch.int32, device=DEV).reshape(batch, 2).contiguous()

    def run(ids, q_out, storage):
        ops.sample_rows_out(logits, cfg, offsets, ids)
        ops.qk_norm_rope_paged_out(q, k, v, gq, gk, pos, wl.EPS, wl.THETA, q_out, storage, 0, tables, pos, 1)

    def fresh():
        return (torch.zeros(batch, dtype=torch.int32, device=DEV), torch.zeros_like(q),
                torch.zeros(1, batch * 2, 2, block_size, kv_heads, dim, dtype=torch.float16, device=DEV))

    eager = fresh()
    run(*eager)                      # also sizes the cached sampler workspace before capture
    torch.cuda.synchronize()
    captured = fresh()
    stream, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            run(*captured)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)
    logits[:, 77] = 1e4              # new inputs, same graph
    k.copy_(h(batch, kv_heads, dim))
    graph.replay()
    again = fresh()
    run(*again)
    torch.cuda.synchronize()
    for a, b in zip(again, captured):
        assert torch.equal(a, b)
    assert captured[0].tolist() == [77] * batch


@pytest.mark.parametrize("batch", [1, 3, 4])
def test_decode_tail_replays_from_a_cuda_graph(b2, port, batch):
    """Final norm + LM head + greedy pick, the tail of the reference's graph-captured decode step
    (src/qwen3_cuda_model.cpp:1069-1071 followed by the argmax of :1339), as two launches in a graph."""
    rng = np.random.default_rng(40 + batch)
    vocab = 20000
    hidden = torch.from_numpy(wl.normal(rng, (batch, 1024), dtype=np.float16)).to(DEV)
    w = torch.from_numpy(wl.gamma(rng, 1024, dtype=np.float16)).to(DEV)
    table = torch.from_numpy(wl.normal(rng, (vocab, 1024), 0.02, np.float16)).to(DEV)
    normed = torch.zeros_like(hidden)
    ids = torch.zeros(batch, dtype=torch.int32, device=DEV)

    def tail():
        ops.cuda_rms_norm_out(hidden, w, wl.EPS, normed)
        ops.lm_head_argmax(normed, table, ids_out=ids)

    tail()                                      # warms the library's per-device state before capture
    torch.cuda.synchronize()
    want = ids.clone()
    ids.zero_()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            tail()
    assert int(ids.abs().sum().item()) == 0     # nothing ran during capture
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ids, want)
    # new hidden rows, same graph; checked against the CPU operators on the normalised rows the graph produced
    hidden.copy_(torch.from_numpy(wl.normal(rng, (batch, 1024), dtype=np.float16)).to(DEV))
    graph.replay()
    torch.cuda.synchronize()
    n32 = port.decode_f16(normed.cpu().numpy().view(np.uint16)).reshape(batch, 1024)
    t32 = port.decode_f16(table.cpu().numpy().view(np.uint16)).reshape(vocab, 1024)
    stored = port.linear(n32, t32).astype(np.float16)
    ours = torch.empty(batch, vocab, dtype=torch.float16, device=DEV)
    assert torch.equal(ops.lm_head_argmax(normed, table, logits_out=ours), ids)
    assert np.array_equal(ids.cpu().numpy(), port.argmax_rows(ours.cpu().numpy().view(np.uint16)))
    close = np.abs(ours.cpu().numpy().astype(np.float64) - stored.astype(np.float64)) <= 2.0 ** -10 * np.maximum(np.abs(stored), 1.0)
    assert close.all()

