"""GPU parity of the decode megakernel against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from flint_b200 import packing
from flint_b200.config import ModelArgs
from flint_b200.engine import DecodeEngine, decode_mega_launch
from oracle import oracle as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 2e-2      # max-abs on logits, the bar stated for the int4 path at the tiny config's logit scale


def logit_tol(ref):
    """2e-2 max-abs is stated on the tiny config, whose largest |logit| is 2.56. Models with larger logits get the
    same RELATIVE bar. (The CPU oracle alone moves by this much when one bf16 ulp of one input element is flipped:
    tests/test_packer_oracle.py::test_oracle_one_ulp_sensitivity.)"""
    return LOGIT_TOL * max(1.0, float(np.abs(ref).max()) / 2.56)


def _to_cuda(P):
    return {k: v.cuda() for k, v in P.items()}


def _run_parity(cfg, P, prompt, steps, max_seq, norm_note=""):
    orc = O.OracleModel(cfg, P, max_seq)
    eng = DecodeEngine(cfg, _to_cuda(P), max_seq=max_seq)
    pos, worst, agree, total = 0, 0.0, 0, 0
    cur = prompt[0]
    seq = list(prompt)
    for i in range(len(prompt) + steps - 1):
        tok = seq[i]
        ref = orc.decode(tok, pos)
        got = eng.decode(tok, pos).cpu().numpy()
        nxt = int(eng.next_token.item())
        eng.check()
        worst = max(worst, float(np.abs(got - ref).max()))
        assert nxt == int(np.argmax(got)), "device argmax must be the first index of the maximum of its own logits"
        if i >= len(prompt) - 1:
            total += 1
            agree += int(nxt == O.argmax_first(ref))
            seq.append(O.argmax_first(ref))          # teacher-forced on the oracle's greedy token
        pos += 1
    kc = eng.kc.cpu().view(torch.int16).numpy().view(np.uint16)
    vc = eng.vc.cpu().view(torch.int16).numpy().view(np.uint16)
    kv_diff = max(np.abs(O.bf16_to_f32(kc[:, :pos]) - O.bf16_to_f32(orc.kc[:, :pos])).max(),
                  np.abs(O.bf16_to_f32(vc[:, :pos]) - O.bf16_to_f32(orc.vc[:, :pos])).max())
    eng.close()
    return worst, agree, total, kv_diff


@pytest.mark.parametrize("asym", [False, True])
def test_tiny_decode_vs_oracle(asym):
    """Tiny config, 16-token prompt + 64 greedy steps: logits within 2e-2 max-abs, >= 99 % greedy agreement."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 0, asym=asym)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=torch.Generator().manual_seed(1234)).tolist()
    worst, agree, total, kv = _run_parity(cfg, P, prompt, 64, cfg.block_size)
    assert worst < LOGIT_TOL, worst
    assert agree >= 0.99 * total, (agree, total)
    assert kv < 0.05, kv


def test_tiny_decode_ref_norm_weights_and_chunked_attention():
    """Norm weights |N(0,1)|+0.5 as the reference's kernel tests use, and the flash-decode split forced to
    2 chunks per kv head so the partial/merge path is exercised at short length."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 1, norm_mode="ref")
    orc = O.OracleModel(cfg, P, 128)
    eng = DecodeEngine(cfg, _to_cuda(P), max_seq=128)
    eng.set_option(1, 3)
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    worst_rel, agree = 0.0, 0
    for pos, t in enumerate(toks):
        ref = orc.decode(t, pos)
        got = eng.decode(t, pos).cpu().numpy()
        worst_rel = max(worst_rel, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
        agree += int(int(eng.next_token.item()) == O.argmax_first(ref))
    eng.check()
    # these norm weights make the logits ~1.3x larger than the unit-norm model the 2e-2 max-abs bar is stated for,
    # so this case uses the reference's own criterion: rel-L2 < 0.02 and equal argmax
    # (reference: bench/verify_mega_test.py:54-56)
    assert worst_rel < 0.02, worst_rel
    assert agree >= len(toks) - 1, agree


def test_reference_shaped_launch_function():
    """decode_mega_launch(...) with the reference's positional arguments (reference: chat.py:71-74)."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 0)
    W = _to_cuda(P)
    orc = O.OracleModel(cfg, P, 64)
    kc = torch.zeros(cfg.n_layer, 64, cfg.n_local_heads, cfg.head_dim, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    for pos, tok in enumerate([7, 300, 4095]):
        h = (W["embed"][tok].float() * cfg.embedding_multiplier).to(torch.bfloat16)
        lg = decode_mega_launch(W["qkv_q"], W["qkv_s"], W["o_q"], W["o_s"], W["n1"], W["gu_q"], W["gu_s"], W["d_q"],
                                W["d_s"], W["n2"], W["nf"], W["lm_q"], W["lm_s"], h, kc, vc, pos, cfg.attn_scale,
                                cfg.rope_base, cfg.residual_multiplier, cfg.logits_scaling)
        ref = orc.decode(tok, pos)
        assert lg.dtype == torch.float32 and tuple(lg.shape) == (cfg.vocab_size,)
        assert np.abs(lg.cpu().numpy() - ref).max() < LOGIT_TOL


def test_chained_device_tokens_match_host_loop():
    cfg = ModelArgs.from_name("tiny")
    W = _to_cuda(packing.synth_packed(cfg, 0))
    a, b = DecodeEngine(cfg, W, max_seq=64), DecodeEngine(cfg, W, max_seq=64)
    tok, host = 11, []
    for pos in range(24):
        a.decode(tok, pos, want_logits=False)
        tok = int(a.next_token.item())
        host.append(tok)
    buf = torch.tensor([[11], [0]], dtype=torch.int32, device="cuda")
    out = torch.zeros(24, dtype=torch.int32, device="cuda")
    cur = buf[0]
    for pos in range(24):
        nxt = out[pos:pos + 1]
        b.decode_chained(cur, pos, nxt)
        cur = nxt
    b.check()
    assert out.tolist() == host


def test_determinism_bitwise():
    """Two contexts give the same bits; so does the hand-over variant that polls the tagged words directly instead of
    waiting for arrival flags first (it changes when data is looked at, never the arithmetic)."""
    cfg = ModelArgs.from_name("tiny")
    W = _to_cuda(packing.synth_packed(cfg, 0))
    outs = []
    for poll in (0, 0, 1):
        e = DecodeEngine(cfg, W, max_seq=32)
        e.set_option(5, poll)
        lg = [e.decode(t, p).clone() for p, t in enumerate([1, 2, 3, 4, 5])]
        e.check()
        outs.append(torch.stack(lg))
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0], outs[2])


def test_wait_runs_out_reports_timeout_and_context_survives():
    """A wait that nothing satisfies: two tensor-parallel ranks live in this process on this GPU, only rank 0 launches.
    Rank 0's own phases complete, then it polls its inbox for rank 1's partial sums, which never arrive: the bounded
    wait runs out, the launch ENDS, the host reads FB_ERR_TIMEOUT with the place it gave up, and the GPU stays usable:
    a fresh single-GPU context decodes correctly afterwards."""
    import ctypes
    from flint_b200 import _lib
    from flint_b200.tp import shard_packed
    cfg = ModelArgs(block_size=32, vocab_size=1024, n_layer=2, n_head=8, n_local_heads=2, dim=512, intermediate_size=1536)
    P = packing.synth_packed(cfg, 0)
    one = DecodeEngine(cfg, _to_cuda(P), max_seq=32)
    ref = one.decode(5, 0).clone()
    one.check()
    ranks = [DecodeEngine(cfg, _to_cuda(shard_packed(P, cfg, r, 2)), max_seq=32, tp_rank=r, tp_size=2) for r in (0, 1)]
    arr = (ctypes.c_void_p * 2)(ranks[0]._ctx, ranks[1]._ctx)
    for e in ranks:
        _lib.check(e.lib.fb_tp_connect_local(e._ctx, arr, 2), "fb_tp_connect_local")
    ranks[0].set_option(0, 20000)              # far above any wait of a healthy launch, milliseconds for the dead one
    ranks[0].decode(5, 0)
    st = ranks[0].status()
    assert st["code"] == _lib.FB_ERR_TIMEOUT, st
    assert st["where"] == 5 and st["layer"] == 0, st       # a tagged-word wait in the first layer's exchange
    for e in ranks:
        e.close()
    again = one.decode(5, 0).clone()
    one.check()
    assert torch.equal(ref, again)
    fresh = DecodeEngine(cfg, _to_cuda(P), max_seq=32)
    assert torch.equal(ref, fresh.decode(5, 0))
    fresh.check()


def test_spin_limit_zero_gives_up_at_once():
    """With a limit of 0 every wait that is not already satisfied gives up: the launch still ends and reports
    FB_ERR_TIMEOUT or, if every wait happened to be satisfied, nothing; either way the next launch is clean."""
    cfg = ModelArgs.from_name("tiny")
    W = _to_cuda(packing.synth_packed(cfg, 0))
    e = DecodeEngine(cfg, W, max_seq=32)
    ref = e.decode(5, 0).clone()
    e.check()
    e.set_option(0, 0)
    e.decode(5, 0)
    st = e.status()
    assert st["code"] in (0, 5), st
    e.set_option(0, 4000000)
    again = e.decode(5, 0).clone()
    e.check()
    assert torch.equal(ref, again)


def test_bad_arguments_are_errors_not_launches():
    from flint_b200 import _lib
    cfg = ModelArgs.from_name("tiny")
    W = _to_cuda(packing.synth_packed(cfg, 0))
    e = DecodeEngine(cfg, W, max_seq=16)
    with pytest.raises(_lib.FlintError) as ei:
        e.decode(3, 16)                       # pos == max_seq
    assert ei.value.code == _lib.FB_ERR_RANGE
    with pytest.raises(_lib.FlintError):
        e.decode(cfg.vocab_size, 0)
    bad = ModelArgs(block_size=64, vocab_size=1000, n_layer=1, n_head=3, n_local_heads=3, dim=384, intermediate_size=1024)
    with pytest.raises(_lib.FlintError) as ei:
        DecodeEngine(bad, _to_cuda(packing.synth_packed(bad, 0)), max_seq=16)
    assert ei.value.code == _lib.FB_ERR_SHAPE


def _granite_shape(n_layer):
    cfg = ModelArgs.from_name("granite-3b-class")
    cfg.n_layer = n_layer
    return cfg


def test_granite3b_shape_two_layers_vs_oracle():
    """Full-size matrices of the headline shape (d 2560, 32/8 heads of 80, FFN 8192, vocab 49160) at a depth of
    2 layers, where bf16 rounding noise has not yet been amplified: the 2e-2 max-abs bar applies."""
    cfg = _granite_shape(2)
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 64)
    eng = DecodeEngine(cfg, W, max_seq=64)
    worst, agree = 0.0, 0
    toks = [17, 40000, 123, 4567, 9, 31000]
    for pos, t in enumerate(toks):
        ref = orc.decode(t, pos)
        got = eng.decode(t, pos).cpu().numpy()
        eng.check()
        worst = max(worst, float(np.abs(got - ref).max()) / logit_tol(ref))
        agree += int(int(eng.next_token.item()) == O.argmax_first(ref))
    assert worst < 1.0, worst
    assert agree == len(toks)


@pytest.mark.parametrize("variant", [0, 2])
def test_long_context_prefilled_cache_vs_oracle(variant):
    """The long-context configuration: K and V caches pre-filled for 32 768 positions with seeded N(0, 1) values (the
    same bf16 bits in the oracle and on the GPU), then decode steps whose attention is split over every CTA and merged.
    Two layers of the 3B-class shape keep the oracle's run time at a few seconds. Both attention variants: the default
    at this length (K/V through the weight ring, tensor pipe) and the scalar one (option 8 = 2)."""
    cfg = _granite_shape(2)
    T0, steps = 32768, 3
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, T0 + 16)
    eng = DecodeEngine(cfg, W, max_seq=T0 + 16)
    eng.set_option(8, variant)
    g = torch.Generator().manual_seed(7)
    kv = torch.randn(2, cfg.n_layer, T0, cfg.n_local_heads, cfg.head_dim, generator=g).bfloat16()
    eng.kc[:, :T0].copy_(kv[0])
    eng.vc[:, :T0].copy_(kv[1])
    orc.kc[:, :T0] = kv[0].view(torch.int16).numpy().view(np.uint16)
    orc.vc[:, :T0] = kv[1].view(torch.int16).numpy().view(np.uint16)
    worst, agree = 0.0, 0
    toks = [17, 40000, 123][:steps]
    for i, t in enumerate(toks):
        ref = orc.decode(t, T0 + i)
        got = eng.decode(t, T0 + i).cpu().numpy()
        eng.check()
        worst = max(worst, float(np.abs(got - ref).max()) / logit_tol(ref))
        tok = int(eng.next_token.item())      # a near-tie may resolve either way: the pick must be within the logit tolerance of the best
        agree += int(tok == O.argmax_first(ref) or ref[tok] >= ref.max() - logit_tol(ref))
    assert worst < 1.0, worst
    assert agree == len(toks)


@pytest.mark.parametrize("T0", [3, 57, 64, 300, 5000])
def test_tiny_long_cache_variant_vs_oracle(T0):
    """The decode variant whose attention streams K/V through the weight ring as tensor copies and multiplies on the tensor
    pipe (the default on one GPU), forced at every cached length: a chunk shorter than one stage, exactly one
    stage, the step's own row inside a stage, many stages per CTA."""
    cfg = ModelArgs.from_name("tiny")
    P = packing.synth_packed(cfg, 0)
    orc = O.OracleModel(cfg, P, T0 + 8)
    eng = DecodeEngine(cfg, {k: v.cuda() for k, v in P.items()}, max_seq=T0 + 8)
    eng.set_option(8, 1)
    g = torch.Generator().manual_seed(11)
    kv = torch.randn(2, cfg.n_layer, T0, cfg.n_local_heads, cfg.head_dim, generator=g).bfloat16()
    eng.kc[:, :T0].copy_(kv[0])
    eng.vc[:, :T0].copy_(kv[1])
    eng.kc[:, T0:].fill_(float("nan"))                 # rows past the cached length must never reach the result
    eng.vc[:, T0:].fill_(float("nan"))
    orc.kc[:, :T0] = kv[0].view(torch.int16).numpy().view(np.uint16)
    orc.vc[:, :T0] = kv[1].view(torch.int16).numpy().view(np.uint16)
    worst, agree = 0.0, 0
    toks = [17, 4000, 123, 9]
    for i, t in enumerate(toks):
        ref = orc.decode(t, T0 + i)
        got = eng.decode(t, T0 + i).cpu().numpy()
        eng.check()
        assert np.isfinite(got).all()
        worst = max(worst, float(np.abs(got - ref).max()) / logit_tol(ref))
        tok = int(eng.next_token.item())
        agree += int(tok == O.argmax_first(ref) or ref[tok] >= ref.max() - logit_tol(ref))
    assert worst < 1.0, worst
    assert agree == len(toks)


def test_granite3b_class_full_depth_vs_oracle():
    """All 40 layers. The seeded N(0, 0.02) model is chaotic under bf16 rounding at this depth: flipping ONE bf16
    ulp of ONE embedding element moves the ORACLE's own logits by 0.15-0.17 max-abs (rel-L2 0.034, measured with
    the oracle alone), so no two summation orders can agree to 2e-2 here. The bound used is 3x that self-sensitivity,
    plus equal greedy tokens."""
    cfg = ModelArgs.from_name("granite-3b-class")
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 64)
    eng = DecodeEngine(cfg, W, max_seq=64)
    worst_rel, agree = 0.0, 0
    toks = [17, 40000, 123, 4567]
    for pos, t in enumerate(toks):
        ref = orc.decode(t, pos)
        got = eng.decode(t, pos).cpu().numpy()
        eng.check()
        worst_rel = max(worst_rel, float(np.linalg.norm(got - ref) / np.linalg.norm(ref)))
        agree += int(int(eng.next_token.item()) == O.argmax_first(ref))
    assert worst_rel < 0.1, worst_rel
    assert agree == len(toks)


@pytest.mark.parametrize("variant", [0, 1])
def test_llama8b_class_shape_two_layers_vs_oracle(variant):
    """The 8B-class shape on ONE GPU (d 4096, 32/8 heads of 128, FFN 14336 = tiles of 2 rows, vocab 128256, untied LM
    head, RoPE base 500000) at a depth of 2 layers against the oracle: the kernel instantiation the tensor-parallel
    configuration is built from. variant 1 forces the long-cache attention (heads of 128: 32 positions per ring stage)."""
    cfg = ModelArgs.from_name("llama-8b-class")
    cfg.n_layer = 2
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 64)
    eng = DecodeEngine(cfg, W, max_seq=64)
    eng.set_option(8, variant)
    worst, agree = 0.0, 0
    toks = [17, 120000, 123, 4567, 9, 31000]
    for pos, t in enumerate(toks):
        ref = orc.decode(t, pos)
        got = eng.decode(t, pos).cpu().numpy()
        eng.check()
        worst = max(worst, float(np.abs(got - ref).max()) / logit_tol(ref))
        tok = int(eng.next_token.item())
        agree += int(tok == O.argmax_first(ref) or ref[tok] >= ref.max() - logit_tol(ref))
    assert worst < 1.0, worst
    assert agree == len(toks)


def test_llama1b_class_shape_two_layers_decode_and_verify_vs_oracle():
    """A fourth model width (d 2048, 32/8 heads of 64, FFN 8192) at a depth of 2 layers: decode against the oracle, then a
    16-node tree verify (this width has no bf16 warp-level GEMM instantiation: the library routes it to the kernels that
    take the width at run time)."""
    from flint_b200.tree import static_tree
    cfg = ModelArgs.from_name("llama-1b-class")
    cfg.n_layer = 2
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    orc = O.OracleModel(cfg, P, 64)
    eng = DecodeEngine(cfg, W, max_seq=64)
    worst, agree = 0.0, 0
    toks = [17, 120000, 123, 4567, 9, 31000]
    for pos, t in enumerate(toks):
        ref = orc.decode(t, pos)
        got = eng.decode(t, pos).cpu().numpy()
        eng.check()
        worst = max(worst, float(np.abs(got - ref).max()) / logit_tol(ref))
        tok = int(eng.next_token.item())
        agree += int(tok == O.argmax_first(ref) or ref[tok] >= ref.max() - logit_tol(ref))
    assert worst < 1.0, worst
    assert agree == len(toks)
    for M in (6, 16):
        parent, depth = static_tree(M)
        amask = O.tree_mask(parent)
        cand = torch.randint(0, cfg.vocab_size, (M,), generator=torch.Generator().manual_seed(M)).tolist()
        ref_lg, _ = orc.verify(cand, len(toks), np.asarray(depth, np.int32), amask)
        lg, _ = eng.verify(cand, len(toks), depth, torch.from_numpy(amask))
        eng.check()
        lg = lg.cpu().numpy()
        rel = max(float(np.linalg.norm(lg[m] - ref_lg[m]) / np.linalg.norm(ref_lg[m])) for m in range(M))
        assert rel < 0.02, rel


def test_granite3b_class_256_greedy_steps_agree_with_oracle():
    """The agreement gate at the configuration it is stated for: all 40 layers, 128-token prompt, 256 greedy steps,
    teacher-forced on the oracle's tokens.

    The seeded N(0, 0.02) model has nearly flat logits and is chaotic under bf16 rounding at this depth: ONE bf16 ulp
    flipped in ONE input element moves the oracle's OWN logits by up to 0.17 (tests/test_packer_oracle.py measures it at
    the tiny scale). A step whose two best logits are closer than that is decided by rounding noise in any
    implementation, the oracle included. So the gate is: on the steps the oracle itself decides (top-2 margin above
    twice that sensitivity) >= 99 % of the device's picks equal the oracle's, and EVERY pick, decided step or not, lies
    within three sensitivities of the oracle's best logit."""
    SENS = 0.17
    cfg = ModelArgs.from_name("granite-3b-class")
    W = packing.synth_packed(cfg, 0, device="cuda")
    P = {k: v.cpu() for k, v in W.items()}
    n_prompt, steps = 128, 256
    orc = O.OracleModel(cfg, P, n_prompt + steps + 1)
    eng = DecodeEngine(cfg, W, max_seq=n_prompt + steps + 1)
    seq = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(1234)).tolist()
    picks = torch.zeros(n_prompt + steps, dtype=torch.int32, device="cuda")
    refs = []
    for pos in range(n_prompt + steps - 1):
        eng.decode(seq[pos], pos, next_token=picks[pos:pos + 1], want_logits=False)
        ref = orc.decode(seq[pos], pos)
        if pos >= n_prompt - 1:
            best = O.argmax_first(ref)
            seq.append(best)
            refs.append(ref)
    eng.check()
    got = picks[n_prompt - 1:n_prompt + steps - 1].tolist()
    assert len(got) == len(refs) == steps
    decided = agree_decided = agree_all = 0
    worst_gap = 0.0
    for tok, ref in zip(got, refs):
        top2 = np.partition(ref, -2)[-2:]
        margin = float(top2[1] - top2[0])
        same = int(tok == O.argmax_first(ref))
        agree_all += same
        worst_gap = max(worst_gap, float(ref.max() - ref[tok]))
        if margin > 2 * SENS:
            decided += 1
            agree_decided += same
    print(f"greedy agreement: {agree_all}/{steps} of all steps, {agree_decided}/{decided} of the decided steps, "
          f"worst gap of a pick to the oracle's best logit {worst_gap:.3f}")
    assert worst_gap <= 3 * SENS, worst_gap
    assert agree_decided >= 0.99 * decided, (agree_decided, decided)
    assert decided >= steps // 8, decided          # the gate must bite on a real share of the steps
