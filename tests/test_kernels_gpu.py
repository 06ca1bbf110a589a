"""Numerics of every sm_100a kernel against the plain PyTorch fp32 reference of the same op."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from autoparallel_b200.ops import cuda_impl, library

    cuda_impl.ensure_loaded()
    return library, cuda_impl


def _ref(name, *args):
    from autoparallel_b200.ops import reference_impls

    cpu = [a.detach().cpu() if isinstance(a, torch.Tensor) else a for a in args]
    return reference_impls[name](*cpu)


def _close(a, b, rtol, atol):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    assert a.shape == b.shape
    err = (a - b).abs().max().item()
    assert torch.allclose(a, b, rtol=rtol, atol=atol), f"max abs err {err}"


GEMM_SHAPES = [
    (128, 256, 64),
    (256, 512, 256),
    (384, 768, 192),
    (1000, 520, 136),  # ragged M, N; K not a multiple of the k-tile
    (64, 128, 4096),
    (4096, 4096, 1024),
    (130, 264, 72),
]


@pytest.mark.parametrize("M,N,K_", GEMM_SHAPES)
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm(K, M, N, K_, ta, tb, out_dtype):
    lib, impl = K
    torch.manual_seed(0)
    a = torch.randn((K_, M) if ta else (M, K_), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, K_) if tb else (K_, N), device="cuda", dtype=torch.bfloat16)
    c = lib.ops.gemm(a, b, ta, tb, out_dtype)
    impl.check_status()
    A = a.float().cpu().t() if ta else a.float().cpu()
    B = b.float().cpu().t() if tb else b.float().cpu()
    ref = A @ B
    tol = 2e-2 if out_dtype == torch.bfloat16 else 1e-3
    _close(c, ref, rtol=tol, atol=tol * (K_ ** 0.5))


@pytest.mark.parametrize("M,N,K_", [(256, 256, 64), (512, 768, 320), (1000, 520, 136), (4096, 4096, 1024), (384, 264, 72)])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("dynamic", [False, True])
def test_gemm_cta_pairs(K, M, N, K_, ta, tb, dynamic):
    """Same GEMM through the two-CTA (cta_group::2) kernel: 256 x 256 tiles split over a CTA pair, with tiles
    dealt statically or handed out at run time; launched twice in a row (the tile counter must come back to zero)."""
    lib, impl = K
    ext = impl.extension()
    torch.manual_seed(2)
    a = torch.randn((K_, M) if ta else (M, K_), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((N, K_) if tb else (K_, N), device="cuda", dtype=torch.bfloat16)
    prev, prev_dyn = ext.gemm_get_pair_mode(), ext.gemm_get_dynamic_tiles()
    ext.gemm_set_pair_mode(True)
    ext.gemm_set_dynamic_tiles(dynamic)
    try:
        c0 = lib.ops.gemm(a, b, ta, tb, torch.float32)
        c = lib.ops.gemm(a, b, ta, tb, torch.float32)
        torch.cuda.synchronize()
        impl.check_status()
    finally:
        ext.gemm_set_pair_mode(prev)
        ext.gemm_set_dynamic_tiles(prev_dyn)
    A = a.float().cpu().t() if ta else a.float().cpu()
    B = b.float().cpu().t() if tb else b.float().cpu()
    _close(c, A @ B, rtol=1e-3, atol=1e-3 * (K_ ** 0.5))
    assert torch.equal(c0, c)


@pytest.mark.parametrize("E,M,N,K_", [(4, 256, 256, 128), (8, 384, 704, 192), (3, 100, 136, 72), (16, 512, 1408, 2048)])
@pytest.mark.parametrize("pair", [True, False])
def test_grouped_gemm(K, E, M, N, K_, pair):
    """Expert GEMMs of a capacity-based MoE layer: forward (B as stored [E,K,N]), dgrad (B^T) and wgrad."""
    lib, impl = K
    ext = impl.extension()
    torch.manual_seed(3)
    a = torch.randn(E, M, K_, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, K_, N, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(E, M, N, device="cuda", dtype=torch.bfloat16)
    prev = ext.gemm_get_pair_mode()
    ext.gemm_set_pair_mode(pair)
    try:
        y = lib.ops.grouped_mm(a, w, False, torch.float32)
        da = lib.ops.grouped_mm(dy, w, True, torch.float32)
        dw = lib.ops.grouped_mm_wgrad(a, dy, torch.float32)
        torch.cuda.synchronize()
        impl.check_status()
    finally:
        ext.gemm_set_pair_mode(prev)
    A, W, DY = a.float().cpu(), w.float().cpu(), dy.float().cpu()
    _close(y, torch.bmm(A, W), 1e-3, 1e-3 * K_ ** 0.5)
    _close(da, torch.bmm(DY, W.transpose(1, 2)), 1e-3, 1e-3 * N ** 0.5)
    _close(dw, torch.bmm(A.transpose(1, 2), DY), 1e-3, 1e-3 * M ** 0.5)


def test_mm_nd_and_wgrad(K):
    lib, impl = K
    torch.manual_seed(1)
    x = torch.randn(2, 192, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    y = lib.ops.mm_nd(x, w, True, torch.bfloat16)
    _close(y, x.float().cpu() @ w.float().cpu().t(), 2e-2, 0.5)
    dy = torch.randn(2, 192, 384, device="cuda", dtype=torch.bfloat16)
    dx = lib.ops.mm_nd(dy, w, False, torch.bfloat16)
    _close(dx, dy.float().cpu() @ w.float().cpu(), 2e-2, 0.5)
    dw = lib.ops.mm_wgrad(dy, x, torch.float32)
    _close(dw, dy.float().cpu().reshape(-1, 384).t() @ x.float().cpu().reshape(-1, 256), 1e-3, 0.05)
    impl.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,D", [(7, 256), (300, 4096), (64, 8192), (33, 1024)])
def test_rms_norm(K, dtype, rows, D):
    lib, _ = K
    torch.manual_seed(0)
    x = torch.randn(rows, D, device="cuda", dtype=dtype)
    w = torch.randn(D, device="cuda", dtype=dtype)
    y, rstd = lib.ops.rms_norm(x, w, 1e-5)
    ry, rr = _ref("rms_norm", x, w, 1e-5)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(y, ry, tol, tol)
    _close(rstd, rr, 1e-5, 1e-5)
    dy = torch.randn_like(x)
    dx, dw = lib.ops.rms_norm_bwd(dy, x, w, rstd)
    rdx, rdw = _ref("rms_norm_bwd", dy, x, w, rstd)
    _close(dx, rdx, tol, tol)
    _close(dw, rdw, tol, tol * 8 if dtype == torch.bfloat16 else 1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rope_swiglu(K, dtype):
    lib, _ = K
    torch.manual_seed(0)
    x = torch.randn(2, 96, 6, 128, device="cuda", dtype=dtype)
    ang = torch.randn(96, 64, device="cuda")
    for conj in (False, True):
        y = lib.ops.rope(x, ang.cos(), ang.sin(), conj)
        _close(y, _ref("rope", x, ang.cos(), ang.sin(), conj), 2e-2 if dtype == torch.bfloat16 else 1e-5, 2e-2 if dtype == torch.bfloat16 else 1e-5)
    a = torch.randn(50, 1408, device="cuda", dtype=dtype)
    b = torch.randn(50, 1408, device="cuda", dtype=dtype)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(lib.ops.swiglu(a, b), _ref("swiglu", a, b), tol, tol)
    dy = torch.randn_like(a)
    da, db = lib.ops.swiglu_bwd(dy, a, b)
    rda, rdb = _ref("swiglu_bwd", dy, a, b)
    _close(da, rda, tol, tol)
    _close(db, rdb, tol, tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,V", [(5, 1024), (37, 128256), (16, 50264)])
def test_cross_entropy(K, dtype, rows, V):
    lib, _ = K
    torch.manual_seed(0)
    logits = (torch.randn(rows, V, device="cuda") * 3).to(dtype)
    labels = torch.randint(0, V, (rows,), device="cuda")
    loss, lse = lib.ops.cross_entropy(logits, labels)
    rl, rlse = _ref("cross_entropy", logits, labels)
    _close(loss, rl, 1e-4, 1e-4)
    _close(lse, rlse, 1e-4, 1e-4)
    dl = torch.randn(rows, device="cuda")
    d = lib.ops.cross_entropy_bwd(dl, logits, labels, lse)
    rd = _ref("cross_entropy_bwd", dl, logits, labels, lse)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    _close(d, rd, tol, 1e-3 if dtype == torch.bfloat16 else 1e-6)


def test_cast_and_embedding_bwd(K):
    lib, _ = K
    x = torch.randn(1000, 33, device="cuda")
    y = lib.ops.dtype_cast(x, torch.bfloat16)
    assert torch.equal(y, x.to(torch.bfloat16))
    assert torch.equal(lib.ops.dtype_cast(y, torch.float32), y.float())
    dy = torch.randn(4, 20, 64, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 50, (4, 20), device="cuda")
    out = lib.ops.embedding_bwd(dy, ids, 50)
    _close(out, _ref("embedding_bwd", dy, ids, 50), 2e-2, 2e-2)


@pytest.mark.parametrize("causal", [True, False])
def test_attention(K, causal):
    lib, _ = K
    torch.manual_seed(0)
    q = torch.randn(2, 256, 8, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, 256, 2, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(2, 256, 2, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    o, lse = lib.ops.attention(q, k, v, causal, scale)
    ro, rlse = _ref("attention", q, k, v, causal, scale)
    _close(o, ro, 2e-2, 2e-2)
    _close(lse, rlse, 1e-2, 1e-2)
    do = torch.randn_like(o)
    dq, dk, dv = lib.ops.attention_bwd(do, q, k, v, o, lse, causal, scale)
    rdq, rdk, rdv = _ref("attention_bwd", do, q, k, v, ro.to(q.dtype), rlse, causal, scale)
    _close(dq, rdq, 5e-2, 5e-2)
    _close(dk, rdk, 5e-2, 5e-2)
    _close(dv, rdv, 5e-2, 5e-2)


@pytest.mark.parametrize("causal,S,Sk,H,Hkv", [(True, 256, 256, 2, 1), (True, 1024, 1024, 4, 2), (False, 256, 384, 2, 2)])
def test_own_attention_forward(K, causal, S, Sk, H, Hkv):
    lib, impl = K
    torch.manual_seed(0)
    q = torch.randn(2, S, H, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(2, Sk, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(2, Sk, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    scale = 128 ** -0.5
    res = impl.attention_forward_own(q, k, v, causal, scale)
    assert res is not None, "shape is inside the kernel's coverage"
    torch.cuda.synchronize()
    impl.check_status()
    o, lse = res
    ro, rlse = _ref("attention", q, k, v, causal, scale)
    _close(o, ro, 2e-2, 2e-2)
    _close(lse, rlse, 1e-2, 1e-2)
    assert impl.attention_forward_own(q[:, :128], k, v, False, scale) is None  # 128 query rows: not covered


def test_wait_that_runs_out_reports_and_leaves_the_context_usable(K):
    """The error path of every peer wait, without a peer: a flag that nothing raises, a short limit.  The kernel
    returns by itself, the host turns the status word into an exception, and the next kernels run normally."""
    import time

    lib, impl = K
    ext = impl.extension()
    torch.cuda.synchronize()
    impl.check_status()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = impl.status_buffer("cuda")
    t0 = time.perf_counter()
    ext.symm_wait_probe(flag, 1, 200, status)  # waits for flag >= 1 for at most 200 ms
    torch.cuda.synchronize()
    assert 0.15 < time.perf_counter() - t0 < 1.5
    with pytest.raises(RuntimeError, match="peer flag"):
        impl.check_status()
    impl.check_status()  # reported once, then cleared
    flag.fill_(3)
    ext.symm_wait_probe(flag, 2, 200, status)  # a flag that IS raised: no wait, no error
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    c = lib.ops.gemm(a, b, False, True, torch.float32)
    torch.cuda.synchronize()
    impl.check_status()
    _close(c, a.float().cpu() @ b.float().cpu().t(), 1e-3, 1e-3 * 128 ** 0.5)


def test_gemm_gives_up_sm_pairs_on_request_and_still_finishes(K):
    """A collective about to launch beside a persistent GEMM asks for SM pairs: that many pairs (at most half of the
    launch) leave early, the rest take over their tiles, the result is unchanged and the requests are used up."""
    lib, impl = K
    ext = impl.extension()
    torch.manual_seed(5)
    a = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    ref = lib.ops.gemm(a, b, False, True, torch.float32)
    prev = ext.gemm_get_dynamic_tiles()
    ext.gemm_set_dynamic_tiles(True)
    try:
        for pairs in (8, 1000, 3):
            ext.gemm_yield_request(pairs)
            c = lib.ops.gemm(a, b, False, True, torch.float32)
            left = ext.gemm_yield_outstanding()
            assert left == 0, left  # every request found a pair (requests are capped at 32, below half the launch)
            assert torch.equal(c, ref)
        c = lib.ops.gemm(a, b, False, True, torch.float32)  # no request: nobody leaves
        assert torch.equal(c, ref) and ext.gemm_yield_outstanding() == 0
        impl.check_status()
    finally:
        ext.gemm_set_dynamic_tiles(prev)


def test_graphed_train_step_matches_eager_steps():
    """Forward + backward + AdamW captured in one CUDA graph and replayed: same losses as the eager loop."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Shard

    from autoparallel_b200 import AutoParallel, ForwardInputs
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug
    from autoparallel_b200.optim import AdamW
    from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
    from autoparallel_b200.ops import cuda_impl
    from autoparallel_b200.runtime.graph_step import GraphedTrainStep
    from conftest import free_port

    own_pg = not dist.is_initialized()
    if own_pg:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        mesh = init_device_mesh("cuda", (1,), mesh_dim_names=("dp",))
        cfg = llama3_debug(dim=256, n_heads=2, n_kv_heads=1, ffn_hidden=512, vocab_size=1024, max_seq_len=256)
        B, S = 2, 256

        def build():
            with torch.device("meta"):
                model = Transformer(cfg)

            def input_fn():
                return ForwardInputs((torch.randint(0, cfg.vocab_size, (B, S)),), {"labels": torch.randint(0, cfg.vocab_size, (B, S))})

            with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32)) as ap:
                ap.add_parameter_memory_constraint()
                ap.add_input_constraints([(Shard(0),)] * 2)
                ap.optimize_placement()
                pm = ap.apply_placement()
            pm.to_empty(device="cuda")
            pm.init_weights(seed=0)
            return pm, AdamW(pm.parameters(), lr=1e-3, emit_bf16=True)

        g = torch.Generator().manual_seed(0)
        batches = [(torch.randint(0, cfg.vocab_size, (B, S), generator=g).cuda(), torch.randint(0, cfg.vocab_size, (B, S), generator=g).cuda())
                   for _ in range(6)]

        def eager(pm, opt, tok, lab):
            loss = pm(tok, labels=lab)
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss.item()

        pm_a, opt_a = build()
        ref = [eager(pm_a, opt_a, *b) for b in batches]
        pm_b, opt_b = build()
        got = [eager(pm_b, opt_b, *b) for b in batches[:2]]  # eager steps first: lazy initialisation stays out of the capture
        step = GraphedTrainStep(pm_b, opt_b, (batches[0][0],), {"labels": batches[0][1]})
        assert step.kernels_per_replay > 0
        opt_b.param_groups[0]["lr"] = 1e-3  # schedules keep working: the kernel reads the rate from device memory
        got += [step(tok, labels=lab).item() for tok, lab in batches[2:]]
        cuda_impl.check_status()
        assert all(abs(a - b) < 2e-2 for a, b in zip(ref, got)), (ref, got)
        assert float(opt_b.state[next(iter(pm_b.parameters()))]["step"]) == len(batches)
    finally:
        if own_pg:
            dist.destroy_process_group()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_forward_and_backward(K, dtype):
    L, _ = K
    torch.manual_seed(0)
    V, D = 1000, 256
    w = torch.randn(V, D, device="cuda", dtype=dtype, requires_grad=True)
    ids = torch.randint(0, V, (3, 77), device="cuda")
    out = L.embedding(w, ids)
    assert torch.equal(out, torch.nn.functional.embedding(ids, w))
    g = torch.randn_like(out)
    out.backward(g)
    ref = torch.zeros(V, D, dtype=torch.float32).index_add_(0, ids.reshape(-1).cpu(), g.reshape(-1, D).float().cpu())
    _close(w.grad, ref, 2e-2 if dtype == torch.bfloat16 else 1e-5, 2e-2 if dtype == torch.bfloat16 else 1e-5)


def test_factory_ops_traced_on_cpu_follow_the_module_to_the_gpu():
    """A region that builds index tensors with ``device=x.device`` is planned on CPU fake tensors; at run time the
    device constant inside the graphs follows the module (the MoE dispatch does exactly this)."""
    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Shard

    from autoparallel_b200 import AutoParallel
    from conftest import free_port

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(32, 32, bias=False)

        def forward(self, x):
            idx = torch.arange(x.shape[0], device=x.device) % 4
            acc = torch.zeros(4, 32, device=x.device, dtype=x.dtype).index_add(0, idx, self.lin(x))
            return acc.sum()

    own_pg = not dist.is_initialized()
    if own_pg:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        mesh = init_device_mesh("cuda", (1,), mesh_dim_names=("dp",))
        with torch.device("meta"):
            m = M()
        with AutoParallel(m, lambda: torch.rand(16, 32), mesh) as ap:
            ap.add_input_constraints([(Shard(0),)])
            ap.optimize_placement()
            pm = ap.apply_placement()
        pm.to_empty(device="cuda")
        with torch.no_grad():
            pm.lin.weight.to_local().copy_(torch.eye(32))
        x = torch.rand(16, 32, device="cuda")
        out = pm(x)
        out.backward()
        assert torch.allclose(out, x.sum(), rtol=1e-4)
        assert pm.lin.weight.grad is not None
    finally:
        if own_pg:
            dist.destroy_process_group()


@pytest.mark.parametrize("rowwise", [False, True])
def test_scaled_mm_on_the_gpu_matches_the_cpu_reference(rowwise):
    """fp8 projection: the CUDA entry (the library's fp8 GEMM, counted as a library call) against the dequantised product."""
    from autoparallel_b200.ops import cuda_impl

    torch.manual_seed(0)
    x, w = torch.randn(256, 512), torch.randn(384, 512)
    f8 = torch.float8_e4m3fn
    if rowwise:
        sx = x.abs().amax(-1, keepdim=True) / 448.0
        sw = w.abs().amax(-1, keepdim=True) / 448.0
    else:
        sx, sw = x.abs().max() / 448.0, w.abs().max() / 448.0
    xq, wq = (x / sx).to(f8), (w / sw).to(f8)
    ref = (xq.float() * sx) @ (wq.float() * sw).t()
    before = cuda_impl.library_fallbacks.get("scaled_mm", 0)
    y = torch.ops.apb200.scaled_mm(xq.cuda(), wq.cuda(), sx.cuda(), sw.cuda(), True, torch.bfloat16)
    assert cuda_impl.library_fallbacks.get("scaled_mm", 0) == before + 1
    assert y.shape == (256, 384) and y.dtype == torch.bfloat16
    err = (y.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 2e-2, err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T,k,E,C,nb,d", [(64, 2, 8, 5, 2, 48), (4096, 8, 64, 700, 4, 256), (96, 3, 7, 100, 1, 40)])
def test_moe_dispatch_kernels_match_the_cpu_formulas(K, dtype, T, k, E, C, nb, d):
    """moe_slots / moe_scatter / moe_gather / moe_gate_grad (csrc/moe_kernels.cu) against the formulas of ops/moe_ops.py,
    with capacities tight enough to drop assignments in the first case."""
    from autoparallel_b200.ops import cuda_impl, moe_ops  # noqa: F401

    torch.manual_seed(0)
    gi = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    src = torch.randn(T, d).to(dtype)
    w = torch.rand(T, k)
    g = torch.randn(T, d).to(dtype)
    before = cuda_impl.library_fallbacks.get("moe_index", 0)
    ops = torch.ops.apb200
    slot_ref = moe_ops._moe_slots(gi, E, C, nb)
    slot = ops.moe_slots(gi.cuda(), E, C, nb)
    assert torch.equal(slot.cpu(), slot_ref)
    buf_ref = moe_ops._moe_scatter(src, slot_ref, w, E, C, nb)
    buf = ops.moe_scatter(src.cuda(), slot, w.cuda(), E, C, nb)
    assert buf.shape == buf_ref.shape and torch.equal(buf.cpu(), buf_ref)
    out_ref = moe_ops._moe_gather(buf_ref.float(), slot_ref, w.to(dtype).float())
    out = ops.moe_gather(buf, slot, w.cuda())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(out.float().cpu(), out_ref, rtol=tol, atol=tol)
    dw_ref = moe_ops._moe_gate_grad(buf_ref, slot_ref, g)
    dw = ops.moe_gate_grad(buf, slot, g.cuda())
    assert dw.dtype == torch.float32 and torch.allclose(dw.cpu(), dw_ref, rtol=1e-3, atol=1e-3 * d ** 0.5)
    assert cuda_impl.library_fallbacks.get("moe_index", 0) == before  # the kernels ran, not the composite formulas
    cuda_impl.check_status()
