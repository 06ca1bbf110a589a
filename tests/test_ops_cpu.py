"""CPU reference implementations of the operator library against PyTorch's own autograd."""
import math
import pytest
import torch
import torch.nn.functional as F

from autoparallel_b200.ops import library as L


def test_rms_norm_matches_torch():
    torch.manual_seed(0)
    x = torch.randn(4, 6, 32, requires_grad=True)
    w = torch.randn(32, requires_grad=True)
    g = torch.randn(4, 6, 32)
    L.rms_norm(x, w, 1e-5).backward(g)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    F.rms_norm(x2, (32,), w2, 1e-5).backward(g)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5)
    assert torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_rope_matches_complex_rotation():
    torch.manual_seed(0)
    x = torch.randn(2, 8, 4, 16, requires_grad=True)
    ang = torch.randn(8, 8)
    y = L.rope(x, ang.cos(), ang.sin())
    xc = torch.view_as_complex(x.detach().reshape(2, 8, 4, 8, 2))
    ref = torch.view_as_real(xc * torch.polar(torch.ones_like(ang), ang)[None, :, None, :]).flatten(3)
    assert torch.allclose(y, ref, atol=1e-5)
    # backward of a rotation is the inverse rotation
    g = torch.randn_like(y)
    y.backward(g)
    assert torch.allclose(x.grad, L.ops.rope(g, ang.cos(), ang.sin(), True), atol=1e-6)


def test_attention_gqa_matches_sdpa():
    torch.manual_seed(0)
    q = torch.randn(2, 16, 4, 8, requires_grad=True)
    k = torch.randn(2, 16, 2, 8, requires_grad=True)
    v = torch.randn(2, 16, 2, 8, requires_grad=True)
    o = L.attention(q, k, v, causal=True)
    g = torch.randn_like(o)
    o.backward(g)
    q2, k2, v2 = (t.detach().clone().requires_grad_() for t in (q, k, v))
    o2 = F.scaled_dot_product_attention(
        q2.transpose(1, 2), k2.transpose(1, 2).repeat_interleave(2, 1), v2.transpose(1, 2).repeat_interleave(2, 1), is_causal=True
    ).transpose(1, 2)
    o2.backward(g)
    for a, b in ((o, o2), (q.grad, q2.grad), (k.grad, k2.grad), (v.grad, v2.grad)):
        assert torch.allclose(a, b, atol=1e-5)


def test_swiglu_and_cross_entropy():
    torch.manual_seed(0)
    a = torch.randn(5, 16, requires_grad=True)
    b = torch.randn(5, 16, requires_grad=True)
    g = torch.randn(5, 16)
    L.swiglu(a, b).backward(g)
    a2, b2 = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    (F.silu(a2) * b2).backward(g)
    assert torch.allclose(a.grad, a2.grad, atol=1e-6) and torch.allclose(b.grad, b2.grad, atol=1e-6)
    lg = torch.randn(7, 11, requires_grad=True)
    lab = torch.randint(0, 11, (7,))
    L.cross_entropy(lg, lab).backward()
    lg2 = lg.detach().clone().requires_grad_()
    F.cross_entropy(lg2, lab).backward()
    assert torch.allclose(lg.grad, lg2.grad, atol=1e-6)


def test_gemm_family_autograd():
    torch.manual_seed(0)
    for ta, tb in ((False, False), (False, True), (True, False), (True, True)):
        a = torch.randn((6, 5) if ta else (5, 6), requires_grad=True)
        b = torch.randn((7, 6) if tb else (6, 7), requires_grad=True)
        g = torch.randn(5, 7)
        L.ops.gemm(a, b, ta, tb, torch.float32).backward(g)
        a2, b2 = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
        ((a2.t() if ta else a2) @ (b2.t() if tb else b2)).backward(g)
        assert torch.allclose(a.grad, a2.grad, atol=1e-5) and torch.allclose(b.grad, b2.grad, atol=1e-5)
    x = torch.randn(2, 3, 6, requires_grad=True)
    w = torch.randn(4, 6, requires_grad=True)
    g = torch.randn(2, 3, 4)
    L.ops.mm_nd(x, w, True, torch.float32).backward(g)
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    (x2 @ w2.t()).backward(g)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_models_run_on_cpu():
    from autoparallel_b200.models.gpt2 import GPT2, gpt2_debug
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug

    m = Transformer(llama3_debug())
    m.init_weights(0)
    t = torch.randint(0, 1024, (2, 32))
    loss = m(t, t)
    loss.backward()
    assert torch.isfinite(loss)
    g = GPT2(gpt2_debug())
    g.init_weights(0)
    t = torch.randint(0, 512, (2, 16))
    assert torch.isfinite(g(t, t))
    assert g.lm_head.weight is g.wte.weight


def test_moe_ops_match_dense_reference_and_are_shard_invariant():
    """slots -> scatter -> grouped GEMM -> gather equals the per-token dense computation, drops included,
    and computing each token block on its own (what a token-sharded plan does) gives the same result."""
    from autoparallel_b200 import ops as K

    T, k, E, C, nb, d = 64, 2, 4, 5, 4, 8
    torch.manual_seed(0)
    gi = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    x = torch.randn(T, d, requires_grad=True)
    gw = torch.rand(T, k, requires_grad=True)
    w = torch.randn(E, d, d, requires_grad=True)
    slot = K.moe_slots(gi, E, C, nb)
    keep = slot < E * C
    assert (~keep).any() and keep.any()  # the capacity is tight enough to drop something
    for b in range(nb):  # every (block, expert) pair holds at most C rows, in arrival order
        sb, gb = slot[b * 16:(b + 1) * 16], gi[b * 16:(b + 1) * 16]
        for e in range(E):
            pos = sb[gb == e]
            pos = pos[pos < E * C] - e * C
            assert pos.tolist() == list(range(len(pos))) and len(pos) <= C
    buf = K.moe_dispatch(x, slot, E, C, nb)
    y = K.grouped_mm(buf.view(E, nb * C, d), w).view(E, nb, C, d)
    out = K.moe_combine(y, slot, gw)
    ref = torch.stack([sum((gw[t, j] * (x[t] @ w[gi[t, j]]) for j in range(k) if keep[t, j]), torch.zeros(d)) for t in range(T)])
    assert torch.allclose(out, ref, atol=1e-5)
    g = torch.randn(T, d)
    grads = torch.autograd.grad(out, (x, gw, w), g)
    rgrads = torch.autograd.grad(ref, (x, gw, w), g)
    for a_, b_ in zip(grads, rgrads):
        assert torch.allclose(a_, b_, atol=1e-4)
    # block by block = rank by rank under Shard(0) tokens / Shard(1) buffer
    parts = []
    for b in range(nb):
        sl = slice(b * 16, (b + 1) * 16)
        s_b = K.moe_slots(gi[sl], E, C, 1)
        assert torch.equal(s_b, slot[sl])
        buf_b = K.moe_dispatch(x[sl], s_b, E, C, 1)
        assert torch.equal(buf_b[:, 0], buf[:, b])
        parts.append(K.moe_combine(y[:, b:b + 1], s_b, gw[sl]))
    assert torch.allclose(torch.cat(parts), out, atol=1e-6)


def test_adamw_bf16_shadow_replaces_the_cast_until_the_parameter_changes():
    from autoparallel_b200.ops import shadow
    from autoparallel_b200.optim import AdamW

    shadow.clear()
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(64, 32))
    opt = AdamW([p], lr=1e-2, emit_bf16=True)
    cast = torch.ops.apb200.dtype_cast
    assert cast(p.detach(), torch.bfloat16).data_ptr() != p.data_ptr()  # nothing published yet: a real cast
    # (the runtime hands the cast a view of the parameter shard: same storage, same version counter)
    p.grad = torch.randn_like(p)
    opt.step()
    before = shadow.hits
    lp = cast(p.detach(), torch.bfloat16)
    assert shadow.hits == before + 1 and torch.equal(lp, p.data.to(torch.bfloat16))
    assert cast(p.detach(), torch.bfloat16).data_ptr() == lp.data_ptr()  # the same buffer every time, no new tensor
    assert cast(p.detach(), torch.float16).dtype == torch.float16 and shadow.hits == before + 2  # other dtypes: ordinary cast
    with torch.no_grad():
        p.mul_(2.0)  # changed outside the optimizer: the shadow is stale and must not be used
    fresh = cast(p.detach(), torch.bfloat16)
    assert shadow.hits == before + 2 and torch.equal(fresh, p.data.to(torch.bfloat16)) and fresh.data_ptr() != lp.data_ptr()
    p.grad = torch.randn_like(p)
    opt.step()  # valid again after the next optimizer step
    assert torch.equal(cast(p.detach(), torch.bfloat16), p.data.to(torch.bfloat16)) and shadow.hits == before + 3
    ref = torch.nn.Parameter(p.data.clone())
    plain = AdamW([ref], lr=1e-2)
    g = torch.randn_like(p)
    p.grad, ref.grad = g.clone(), g.clone()
    opt.state[p]["step"].zero_(); opt.state[p]["exp_avg"].zero_(); opt.state[p]["exp_avg_sq"].zero_()
    opt.step(); plain.step()
    assert torch.allclose(p.data, ref.data)  # emitting the shadow does not change the update
    shadow.clear()


def test_yarn_rope_tables_keep_fast_pairs_and_stretch_slow_ones():
    from autoparallel_b200.models.llama3 import rope_tables

    d, n, theta = 64, 4096, 10000.0
    cos0, sin0 = rope_tables(d, n, theta)
    cos1, sin1 = rope_tables(d, n, theta, yarn={"factor": 4.0, "original_max_seq_len": 1024, "mscale": 1.0})
    scale = 0.1 * math.log(4.0) + 1.0
    assert cos1.shape == cos0.shape == (n, d // 2)
    # the fastest pair keeps its frequency (only the temperature differs) ...
    assert torch.allclose(cos1[:, 0] / scale, cos0[:, 0], atol=1e-5) and torch.allclose(sin1[:, 0] / scale, sin0[:, 0], atol=1e-5)
    # ... the slowest pair is interpolated: position p of the extended context lands where p / 4 used to
    p = torch.arange(0, n, 4)
    assert torch.allclose(sin1[p, -1] / scale, sin0[p // 4, -1], atol=1e-4)
    # factor 1 (or no yarn) is the plain table
    c, s_ = rope_tables(d, n, theta, yarn={"factor": 1.0})
    assert torch.equal(c, cos0) and torch.equal(s_, sin0)


@pytest.mark.parametrize("causal,mask", [(True, None), (False, None), (False, "float"), (True, "float")])
def test_device_neutral_attention_matches_the_planning_hosts_operator(causal, mask, monkeypatch):
    """``runtime/portable_ops.py``: the stand-ins that replace the CPU-only attention operators when a graph moves to another
    device compute the same outputs, log-sum-exp and gradients (their generic branch is forced here)."""
    from autoparallel_b200.runtime import portable_ops as P

    torch.manual_seed(0)
    B, H, L, D = 2, 3, 16, 8
    q, k, v, go = (torch.randn(B, H, L, D, dtype=torch.float64) for _ in range(4))
    m = None
    if mask == "bool":
        m = torch.rand(B, 1, L, L) > 0.3
        m[..., 0] = True  # no row fully masked
    elif mask == "float":
        m = torch.randn(B, 1, L, L, dtype=torch.float64)
    aten = torch.ops.aten
    ro, rl = aten._scaled_dot_product_flash_attention_for_cpu(q, k, v, 0.0, causal, attn_mask=m)
    rdq, rdk, rdv = aten._scaled_dot_product_flash_attention_for_cpu_backward(go, q, k, v, ro, rl, 0.0, causal, attn_mask=m)
    monkeypatch.setattr(P, "FORCE_GENERIC", True)
    for formulas in (True, False):  # explicit formulas; the library call with a recomputing backward
        monkeypatch.setattr(P, "FORMULAS_ONLY", formulas)
        o, l = P.sdpa_forward(q, k, v, 0.0, causal, attn_mask=m)
        assert torch.allclose(o, ro, atol=1e-9)
        if formulas:
            assert torch.allclose(l.to(rl.dtype), rl, atol=1e-6)
        dq, dk, dv = P.sdpa_backward(go, q, k, v, o, l.double(), 0.0, causal, attn_mask=m)
        assert torch.allclose(dq, rdq, atol=1e-8) and torch.allclose(dk, rdk, atol=1e-8) and torch.allclose(dv, rdv, atol=1e-8)
