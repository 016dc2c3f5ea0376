"""The engine at real Qwen3 layer sizes (hidden 4096, 32/8 heads of 128, intermediate 12288,
vocabulary 151936; two layers so it stays quick) with random weights, against the plain
implementation run in float64 on the GPU, under different ways of cutting the work."""
import pytest
import torch

from tests import replay

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

CFG = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096,
           num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
           vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=512,
           tie_word_embeddings=False)


@pytest.fixture(scope="module")
def setup():
    from leone_b200.config.qwen3 import Qwen3Config
    from leone_b200.engine.model import weight_specs_for_config
    from leone_b200.registry import spec_from_config
    from leone_b200.weights.random_init import draw
    config = Qwen3Config.from_dict(CFG)
    specs = weight_specs_for_config(config)
    tensors = {s.name: draw(s, 5, DEV) for s in specs}
    return config, spec_from_config(config), tensors


def _plain_logits(tensors, tokens, as_bf16):
    from tests.plain import model as pm
    w = {}
    for name, t in tensors.items():
        t = t.to(torch.bfloat16).float() if (as_bf16 and t.dim() == 2) else t
        w[name] = t.double()
    return pm.forward_logits(CFG, w, tokens)


@pytest.mark.parametrize("dtype,rtol,atol_scale,fusions", [("float32", 3e-5, 3e-5, True), ("bfloat16", 3e-2, 3e-2, True),
                                                            ("bfloat16", 3e-2, 3e-2, False)])
def test_real_layer_sizes_under_cuts(setup, dtype, rtol, atol_scale, fusions):
    """``fusions=False``: the same with the cluster reductions, the folded norms, the fused decode
    preparation and the tcgen05 prompt attention switched off, i.e. the kernels that other sizes
    fall back to."""
    from leone_b200.engine.engine import Engine
    config, spec, tensors = setup
    # 300 tokens: the prompt-sized kernels; 45: the decode-sized ones; 150: between them, where the
    # wide gate/up product takes the token-major form and the others the swapped one
    reqs = {"a": replay.random_tokens(151936, 300, 1), "b": replay.random_tokens(151936, 45, 2),
            "c": replay.random_tokens(151936, 150, 3)}
    want = {r: _plain_logits(tensors, t, dtype == "bfloat16").cpu() for r, t in reqs.items()}

    class Plain:
        def logits(self, tokens):
            return want[{300: "a", 45: "b", 150: "c"}[len(tokens)]]

    traces = {"whole": replay.trace_whole(reqs), "tail": replay.trace_decode_tail(reqs, tail=8),
              "mixed": replay.trace_mixed(reqs, seed=1)}
    for name, steps in traces.items():
        # only some positions are wanted: full-vocabulary logits for every row would be large
        for st in steps:
            for e in st["entries"]:
                e["want"] = [w for w in e["want"] if w % 7 == 0 or w == len(e["tokens"]) - 1]
        engine = Engine(spec, dict(tensors), dtype=dtype, page_tokens=16, max_tokens=replay.max_live_tokens(steps),
                        max_requests=4, max_batch_tokens=320)
        if not fusions:
            fast = engine.ops.fast
            fast.use_clusters = fast.fuse_norm = fast.fuse_decode = fast.use_tc_attention = fast.use_token_major = False
        out = replay.run_trace_engine(engine, steps)
        replay.compare(steps, out, Plain(), reqs, rtol, atol_scale, f"8B layer sizes {dtype} {name} fusions={fusions}")
        del engine
        torch.cuda.empty_cache()
