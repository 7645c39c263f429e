"""Parity of the decode step at the REAL benchmark shapes (TinyLlama-1.1B, Llama-3.2-1B, Llama-3-8B, the 8B
shape over a 32768-position cache) and over every attention kernel instantiation, through the C ABI
against the CPU oracle on identical seeded weights and teacher-forced tokens.

Tolerances are the task's: per-step logits max-abs <= 2e-2 and cosine >= 0.9999 for FP16 weights; sampled
ids compared on IDENTICAL logits, history and r.  The oracle reads the binary16 weights as they are (exact
widening on use), so the 8B shape needs about 16 GB of host memory for the weights instead of 32."""
import numpy as np
import pytest

from lighterpp_b200 import synth
from lighterpp_b200.formats import ModelConfig

pytestmark = pytest.mark.gpu

FP16_MAX_ABS, FP16_MIN_COS, FP32_MAX_ABS = 2e-2, 0.9999, 1e-4


@pytest.fixture(scope="module")
def E():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from lighterpp_b200 import engine
    return engine


def mem_available_gb() -> float:
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) / 1e6
    except OSError:
        pass
    return 0.0


def check_logits(ref, got, dt="f16"):
    d = float(np.abs(ref - got).max())
    cos = float(np.dot(ref, got) / (np.linalg.norm(ref) * np.linalg.norm(got)))
    if dt == "f32":
        assert d <= FP32_MAX_ABS, d
    else:
        assert d <= FP16_MAX_ABS and cos >= FP16_MIN_COS, (d, cos)
    return d, cos


def teacher_forced(eng, m, oracle, c, prompt, n_steps, temp, pen, rs, dt="f16", start_pos=0):
    """n_steps steps at start_pos..: the prompt first, then the oracle's own sampled tokens.  Every step compares
    logits and, on the oracle's logits, the sampled id for argmax and for (temp, pen) with the step's r."""
    hist, worst, worst_cos = [], 0.0, 1.0
    tok = int(prompt[0])
    for i in range(n_steps):
        pos = start_pos + i
        hist = (hist + [tok])[-64:]
        ref = m.step_logits(tok, pos)
        got = eng.step_logits(tok, pos)
        d, cos = check_logits(ref, got, dt)
        worst, worst_cos = max(worst, d), min(worst_cos, cos)
        assert eng.sample(ref, 0.0, pen, hist, 0.0) == oracle.sample(ref, 0.0, pen, hist, 0.0), pos
        want = oracle.sample(ref, temp, pen, hist, float(rs[i]))
        assert eng.sample(ref, temp, pen, hist, float(rs[i])) == want, (pos, float(rs[i]))
        tok = int(prompt[i + 1]) if i + 1 < len(prompt) else want
    return worst, worst_cos


def test_tinyllama_shape_16_steps(E, oracle):
    """Config 2 (32 query heads on 4 KV heads: the 8-heads-per-KV-head attention kernel), 16 teacher-forced steps."""
    c, dt, tied, seed = synth.SHAPES["tinyllama-1.1b"]
    c = ModelConfig(**{**c.asdict(), "seq_len": 64})
    T = synth.gen_model(c, seed, dt, tied, threads=8)
    eng = E.Engine(c, dt, "f16")
    eng.load_weights(T)
    m = oracle.model(c, T, keep_f16=True)
    prompt = synth.prompt_tokens(c.vocab_size, 12, seed)
    worst, cos = teacher_forced(eng, m, oracle, c, prompt, 16, 0.8, 1.1, oracle.rand_floats(1234, 16))
    print(f"tinyllama-1.1b shape, 16 steps: worst max-abs {worst:.2e}, worst cosine {cos:.7f}")
    eng.close()


def test_llama32_1b_shape_64_steps(E, oracle):
    """Config 3 (128K vocabulary, tied classifier, penalty 1.1, temperature 0.8): 64 teacher-forced steps."""
    c, dt, tied, seed = synth.SHAPES["llama-3.2-1b"]
    c = ModelConfig(**{**c.asdict(), "seq_len": 128})
    T = synth.gen_model(c, seed, dt, tied, threads=8)
    eng = E.Engine(c, dt, "f16")
    eng.load_weights(T)
    m = oracle.model(c, T, keep_f16=True)
    prompt = synth.prompt_tokens(c.vocab_size, 32, seed)
    worst, cos = teacher_forced(eng, m, oracle, c, prompt, 64, 0.8, 1.1, oracle.rand_floats(1234, 64))
    print(f"llama-3.2-1b shape, 64 steps: worst max-abs {worst:.2e}, worst cosine {cos:.7f}")
    eng.close()


def test_llama3_8b_shape_short_and_32k_context(E, oracle):
    """Configs 4 and 5 on one GPU: the Llama-3-8B shape (64-bit weight offsets, 14336-wide down projection, head
    size 128), 8 teacher-forced steps from position 0, then the K/V cache pre-filled with 32768 positions of seeded
    N(0,1) FP16 values and 4 more steps from position 32768 (every KV split in use)."""
    if mem_available_gb() < 40:
        pytest.skip("needs about 40 GB of free host memory for the 8B weights and the oracle's FP32 cache")
    c, dt, tied, seed = synth.SHAPES["llama-3-8b"]
    n_pre = 32768
    c = ModelConfig(**{**c.asdict(), "seq_len": n_pre + 8})
    T = synth.gen_model(c, seed, dt, tied, threads=16)
    eng = E.Engine(c, dt, "f16")
    eng.load_weights(T)
    m = oracle.model(c, T, keep_f16=True)
    prompt = synth.prompt_tokens(c.vocab_size, 64, seed)
    worst, cos = teacher_forced(eng, m, oracle, c, prompt, 8, 0.8, 1.1, oracle.rand_floats(1234, 8))
    print(f"llama-3-8b shape, 8 steps from position 0: worst max-abs {worst:.2e}, worst cosine {cos:.7f}")
    # long context: the cache rows of positions 0..n_pre-1 are overwritten on both sides with the same values
    ko, vo = m.kv_cache()
    for l in range(c.n_layers):
        rng = np.random.default_rng([4, l])
        k = rng.standard_normal((c.n_kv_heads, n_pre, c.head_size), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((c.n_kv_heads, n_pre, c.head_size), dtype=np.float32).astype(np.float16)
        ko[l, :, :n_pre] = k
        vo[l, :, :n_pre] = v
        eng.kv_prefill(l, k, v, n_pre)
    worst, cos = teacher_forced(eng, m, oracle, c, prompt[8:], 4, 0.8, 1.1, oracle.rand_floats(4321, 4), start_pos=n_pre)
    print(f"llama-3-8b shape, 4 steps from position {n_pre}: worst max-abs {worst:.2e}, worst cosine {cos:.7f}")
    eng.close()


# head size x query heads per KV head: the eight tensor-core instantiations, the CUDA-core kernel for the head
# sizes the tensor-core kernel does not take, and the FP32 cache
ATTN_CASES = [(hs, g, "f16") for hs in (64, 128) for g in (1, 2, 4, 8)] + \
             [(48, 2, "f16"), (96, 4, "f16"), (64, 4, "f32"), (128, 8, "f32"), (32, 1, "f16"), (16, 2, "f32")]


@pytest.mark.parametrize("hs,gqa,kv", ATTN_CASES)
def test_every_attention_instantiation(E, oracle, hs, gqa, kv):
    """Toy-width models that differ only in the attention geometry; first positions (one partly filled tile, one
    split) and, behind a pre-filled cache of 700 positions, several splits with a ragged last tile."""
    n_kv = 2
    n_heads = n_kv * gqa
    c = ModelConfig(n_heads * hs, 256, 2, n_heads, n_kv, 512, 720, 500000.0)
    seed = 1000 + hs * 16 + gqa
    T = synth.gen_model(c, seed, "f16", True)
    eng = E.Engine(c, "f16", kv)
    eng.load_weights(T)
    m = oracle.model(c, synth.as_f32(T))
    toks = synth.prompt_tokens(c.vocab_size, 9, seed)
    for pos in range(5):
        check_logits(m.step_logits(int(toks[pos]), pos), eng.step_logits(int(toks[pos]), pos))
    n_pre = 700
    rng = np.random.default_rng(seed)
    ko, vo = m.kv_cache()
    for l in range(c.n_layers):
        k = rng.standard_normal((n_kv, n_pre, hs)).astype(np.float16)
        v = rng.standard_normal((n_kv, n_pre, hs)).astype(np.float16)
        ko[l, :, :n_pre] = k
        vo[l, :, :n_pre] = v
        conv = np.float16 if kv == "f16" else np.float32
        eng.kv_prefill(l, k.astype(conv), v.astype(conv), n_pre)
    for i in range(4):
        pos = n_pre + i
        check_logits(m.step_logits(int(toks[5 + i]), pos), eng.step_logits(int(toks[5 + i]), pos))
    # the K/V rows those steps wrote sit at the reference's index
    tol = 2e-3 if kv == "f16" else 1e-5
    for l in range(c.n_layers):
        for h in range(n_kv):
            k, v = eng.kv_read(l, h, n_pre + 3)
            assert np.abs(k - ko[l, h, n_pre + 3]).max() < tol * max(1.0, np.abs(ko[l, h, n_pre + 3]).max())
            assert np.abs(v - vo[l, h, n_pre + 3]).max() < tol * max(1.0, np.abs(vo[l, h, n_pre + 3]).max())
    eng.close()
