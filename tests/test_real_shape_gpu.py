"""The engine at real Qwen3 layer sizes (the 8B, 32B and 1.7B layer shapes over the full
vocabulary of 151,936; two layers so it stays quick) with seeded random weights, against the
plain implementation run in float64 on the GPU, under every way of cutting the work.  The
engine is made by ``Engine.from_config`` (weights drawn on the device); the plain side gets
the same values from the same definition of the draw (``tests/test_random_weights.py`` checks
the device draw against the host draw and the tests' numpy restatement bit for bit)."""
import pytest
import torch

from tests import replay

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
VOCAB = 151936

SHAPES = {
    # the headline shape: n_q * d == hidden
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, tie_word_embeddings=False),
    # n_q * d = 8192 != hidden; group of 8; the widest feed-forward
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                intermediate_size=25600, tie_word_embeddings=False),
    # group of 2; the head reads the embedding table
    "1.7b": dict(hidden_size=2048, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                 intermediate_size=6144, tie_word_embeddings=True),
}
SEED = 5


def _cfg(shape, positions=512):
    return dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, vocab_size=VOCAB, rope_theta=1000000.0,
                rms_norm_eps=1e-6, max_position_embeddings=positions, **SHAPES[shape])


def _plain_weights(cfg):
    from leone_b200.config.qwen3 import Qwen3Config
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.weights.random_init import draw
    specs = weight_specs_for_config(Qwen3Config.from_dict(cfg))
    return {s.name: draw(s, SEED, DEV) for s in specs}


def _plain_logits(cfg, tensors, tokens, as_bf16):
    from tests.plain import model as pm
    w = {}
    for name, t in tensors.items():
        t = t.to(torch.bfloat16).float() if (as_bf16 and t.dim() == 2) else t
        w[name] = t.double()
    return pm.forward_logits(cfg, w, tokens)


@pytest.fixture(scope="module", params=list(SHAPES))
def setup(request):
    from leone_b200.config.qwen3 import Qwen3Config
    shape = request.param
    cfg = _cfg(shape)
    tensors = _plain_weights(cfg)
    # 300 tokens: the prompt-sized kernels; 45: the decode-sized ones; 150: between them, where the
    # wide gate/up product takes the token-major form and the others the swapped one
    # 400 (its own test): products on pairs of SMs with the norms folded into them
    reqs = {"a": replay.random_tokens(VOCAB, 300, 1), "b": replay.random_tokens(VOCAB, 45, 2),
            "c": replay.random_tokens(VOCAB, 150, 3), "d": replay.random_tokens(VOCAB, 400, 4)}
    want = {}
    for bf in (False, True):
        for r, t in reqs.items():
            want[(bf, r)] = _plain_logits(cfg, tensors, t, bf).cpu()
    del tensors
    torch.cuda.empty_cache()
    return shape, cfg, Qwen3Config.from_dict(cfg), reqs, want


@pytest.mark.parametrize("dtype,fusions", [("float32", True), ("bfloat16", True), ("bfloat16", False)])
def test_real_layer_sizes_under_cuts(setup, dtype, fusions):
    """``fusions=False``: the same with the cluster reductions, the folded norms, the fused decode
    preparation and the tcgen05 prompt attention switched off, i.e. the kernels that other sizes
    fall back to."""
    from leone_b200.engine.engine import Engine
    shape, cfg, config, reqs, want = setup
    reqs = {r: reqs[r] for r in "abc"}
    bf = dtype == "bfloat16"

    class Plain:
        def logits(self, tokens):
            return want[(bf, {300: "a", 45: "b", 150: "c"}[len(tokens)])]

    traces = {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=32),
              "portions": replay.trace_portions(reqs, sizes=(130, 2, 37, 70, 5, 3, 2, 33, 1, 16)),
              "mixed": replay.trace_mixed(reqs, seed=1)}
    for name, steps in traces.items():
        # only some positions are wanted: full-vocabulary logits for every row would be large
        for st in steps:
            for e in st["entries"]:
                e["want"] = [w for w in e["want"] if w % 7 == 0 or w == len(e["tokens"]) - 1]
        engine = Engine.from_config(config, SEED, dtype=dtype, page_tokens=16, max_tokens=replay.max_live_tokens(steps),
                                    max_requests=4, max_batch_tokens=320)
        if not fusions:
            fast = engine.ops.fast
            fast.use_clusters = fast.fuse_norm = fast.fuse_decode = fast.use_tc_attention = fast.use_token_major = False
        out = replay.run_trace_engine(engine, steps)
        what = f"{shape} layer sizes {dtype} {name} fusions={fusions}"
        # 32-bit: sums of up to 25,600 products in another order than the float64 side's
        tol = (3e-5, 3e-5) if dtype == "float32" else replay.tolerance(dtype)
        worst = replay.compare(steps, out, Plain(), reqs, *tol, what)
        replay.check_worst(("real", shape, dtype, name, fusions), worst)
        del engine
        torch.cuda.empty_cache()


def test_real_layer_sizes_a_prompt_on_pairs_of_sms(setup):
    """A prompt of 400 tokens in one step (every product of the layers on pairs of SMs, with the
    norms folded into them), and in portions of 385 and 15; a short request after it."""
    from leone_b200.engine.engine import Engine
    shape, cfg, config, reqs, want = setup
    reqs = {r: reqs[r] for r in "db"}

    class Plain:
        def logits(self, tokens):
            return want[(True, {400: "d", 45: "b"}[len(tokens)])]

    for name, steps in {"whole": replay.trace_whole(reqs),
                        "portions": replay.trace_portions(reqs, sizes=(385, 15, 2, 43))}.items():
        for st in steps:
            for e in st["entries"]:
                e["want"] = [w for w in e["want"] if w % 7 == 0 or w == len(e["tokens"]) - 1]
        engine = Engine.from_config(config, SEED, dtype="bfloat16", page_tokens=16,
                                    max_tokens=replay.max_live_tokens(steps), max_requests=4, max_batch_tokens=448)
        if not engine.ops.fast.use_pairs:
            pytest.skip("LEONE_NO_PAIRS is set")
        assert engine.ops.fast.in_pairs(400) and engine.ops.fast.fuses_norm(400)
        out = replay.run_trace_engine(engine, steps)
        worst = replay.compare(steps, out, Plain(), reqs, *replay.tolerance("bfloat16"),
                               f"{shape} layer sizes, 400 tokens on pairs, {name}")
        replay.check_worst(("real-pairs", shape, name), worst)
        del engine
        torch.cuda.empty_cache()


@pytest.mark.parametrize("context", [5, 130, 2100])
def test_decode_graph_at_the_models_real_position_limit(context):
    """A real ``config.json`` allows 40,960 positions.  The captured decode step must give the
    eager step's tokens and logits there from short and long contexts alike (its split counts
    and table widths are chosen from the live lengths, not from the limit)."""
    from leone_b200.config.qwen3 import Qwen3Config
    from leone_b200.engine.engine import Engine
    from leone_b200.sampling.sampler import SamplingParams
    config = Qwen3Config.from_dict(_cfg("8b", positions=40960))
    batch = 3
    prompts = [replay.random_tokens(VOCAB, context + i, 40 + i) for i in range(batch)]
    results = []
    for use_graph in (False, True):
        eng = Engine.from_config(config, SEED, dtype="bfloat16", page_tokens=16, max_tokens=batch * (context + 64),
                                 max_requests=batch, max_batch_tokens=1024)
        for i, p in enumerate(prompts):
            for at in range(0, len(p) - 1, 1024):
                eng.step([(i, p[at:min(at + 1024, len(p) - 1)], [])])
        params = [SamplingParams() for _ in range(batch)]
        last = [p[-1] for p in prompts]
        toks = []
        if use_graph:
            toks += eng.decode_steps(range(batch), last, params, 4)          # a quantum
            for _ in range(3):                                                # single steps, launched ahead
                toks += eng.decode_steps(range(batch), toks[-1], params, 1)
            logits = eng.decode_logits(range(batch), toks[-1]).clone()
        else:
            for _ in range(7):
                lg = eng.step([(i, [t], [0]) for i, t in enumerate(last)])
                last = eng.sample(lg, params, [eng.length(i) - 1 for i in range(batch)])
                toks.append(last)
            logits = eng.step([(i, [t], [0]) for i, t in enumerate(last)])
        results.append((toks, logits.float().cpu()))
        del eng
        torch.cuda.empty_cache()
    (eager_toks, eager_logits), (graph_toks, graph_logits) = results
    # greedy ids may differ only where two logits tie within rounding: compare the logits, and
    # the ids wherever the eager step's lead is clear
    scale = eager_logits.abs().max().item()
    if graph_toks == eager_toks:
        assert (graph_logits - eager_logits).abs().max().item() <= 2e-2 * scale
    else:
        first = next(i for i, (a, b) in enumerate(zip(graph_toks, eager_toks)) if a != b)
        pytest.fail(f"graph and eager decode differ at step {first}: {graph_toks[first]} vs {eager_toks[first]}")
