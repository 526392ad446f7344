"""sm_100a kernels versus plain PyTorch fp32 references (run on a B200)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _random_csr(rows, cols, mean_deg, long_row=None, empty_every=7, seed=0):
    g = torch.Generator().manual_seed(seed)
    deg = torch.poisson(torch.full((rows,), float(mean_deg)), generator=g).long().clamp(max=cols)
    deg[::empty_every] = 0
    if long_row is not None:
        deg[long_row[0]] = min(cols, long_row[1])
    crow = torch.zeros(rows + 1, dtype=torch.int64)
    crow[1:] = torch.cumsum(deg, 0)
    nnz = int(crow[-1])
    col = torch.empty(nnz, dtype=torch.int64)
    for r in range(rows):
        d = int(deg[r])
        if d:
            col[crow[r]:crow[r + 1]] = torch.randperm(cols, generator=g)[:d].sort().values
    val = torch.randn(nnz, generator=g)
    return torch.sparse_csr_tensor(crow.int(), col.int(), val, size=(rows, cols), check_invariants=False)


# 1: CUDA-core kernel, 2: tensor-core kernel
@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("D", [8, 24, 48, 104, 128, 256, 304, 608])
def test_spmm_bf16_matches_fp32_reference(D, variant):
    from plexus_b200.ops import cuda as opc

    A = _random_csr(700, 500, 9, long_row=(13, 5000 if D < 300 else 450), seed=D)
    H = torch.randn(500, D)
    Hb = H.to(torch.bfloat16)
    ref = torch.sparse.mm(A, Hb.float())
    out = opc.spmm(A.to(_dev()), Hb.to(_dev()), variant=variant)
    opc.check_status()
    assert out.dtype == torch.bfloat16
    err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 1e-2, err
    # every row, not only the largest one
    scale = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-3)
    assert ((out.float().cpu() - ref).abs() / scale).max() < 3e-2


def test_spmm_long_rows_and_mask_and_row_range():
    from plexus_b200 import ops

    rows, cols, D = 300, 9000, 128
    A = _random_csr(rows, cols, 20, long_row=(5, 8000), seed=1)
    H = torch.randn(cols, D).to(torch.bfloat16)
    mask = torch.randn(rows, D).to(torch.bfloat16)
    ref = torch.sparse.mm(A, H.float())
    Ad, Hd = A.to(_dev()), H.to(_dev())
    full = ops.spmm(Ad, Hd).float().cpu()
    assert (full - ref).abs().max() / ref.abs().max() < 1e-2
    masked = ops.spmm(Ad, Hd, relu_mask=mask.to(_dev())).float().cpu()
    want = ref * (mask.float() > 0)
    assert (masked - want).abs().max() / ref.abs().max() < 1e-2
    part = ops.spmm(Ad, Hd, row_range=(3, 111)).float().cpu()
    assert (part - ref[3:111]).abs().max() / ref.abs().max() < 1e-2


def _csr_from_degrees(deg, cols, seed):
    g = torch.Generator().manual_seed(seed)
    rows = deg.numel()
    crow = torch.zeros(rows + 1, dtype=torch.int64)
    crow[1:] = torch.cumsum(deg, 0)
    nnz = int(crow[-1])
    col = torch.randint(0, cols, (nnz,), generator=g)
    val = torch.randn(nnz, generator=g)
    return torch.sparse_csr_tensor(crow.int(), col.int(), val, size=(rows, cols), check_invariants=False)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("D", [16, 48, 56, 104, 128, 256])
def test_spmm_row_patterns(D, variant):
    """Runs of tiny rows (several rows per 16-nonzero stage, more than four: forced flushes inside a
    stage), empty rows at the start, in the middle and at the end, rows that end exactly on a stage
    boundary, one long row (whole, and cut in pieces that different warps sum), a mask and a row range."""
    from plexus_b200.ops import cuda as opc

    g = torch.Generator().manual_seed(D)
    cols = 3000
    deg = torch.cat([
        torch.zeros(5, dtype=torch.long),                      # leading empty rows
        torch.randint(0, 4, (400,), generator=g),              # tiny rows, some empty
        torch.full((40,), 16, dtype=torch.long),               # rows ending on stage boundaries
        torch.randint(1, 3, (300,), generator=g),
        torch.tensor([2500, 0, 0, 1, 33, 0]),                  # a long row among empty ones
        torch.randint(20, 60, (500,), generator=g),            # typical rows
        torch.zeros(9, dtype=torch.long),                      # trailing empty rows
    ])
    A = _csr_from_degrees(deg, cols, seed=D + 1)
    rows = deg.numel()
    H = torch.randn(cols, D, generator=g).to(torch.bfloat16)
    mask = torch.randn(rows, D, generator=g).to(torch.bfloat16)
    ref = torch.sparse.mm(A, H.float())
    scale = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-3)
    Ad, Hd = A.to(_dev()), H.to(_dev())
    for block_cost, long_row in ((64, 200), (4096, 4096), (512, 16)):
        saved = opc.SPMM_BLOCK_COST[variant], opc.SPMM_LONG_ROW[variant]
        opc.SPMM_BLOCK_COST[variant], opc.SPMM_LONG_ROW[variant] = block_cost, long_row
        try:
            out = opc.spmm(Ad, Hd, variant=variant).float().cpu()
            opc.check_status()
            assert ((out - ref).abs() / scale).max() < 3e-2, block_cost
            assert float(out[deg == 0].abs().max()) == 0.0
            masked = opc.spmm(Ad, Hd, relu_mask=mask.to(_dev()), variant=variant).float().cpu()
            assert (((masked - ref * (mask.float() > 0)).abs()) / scale).max() < 3e-2
            part = opc.spmm(Ad, Hd, row_range=(3, 777), variant=variant).float().cpu()
            assert ((part - ref[3:777]).abs() / scale[3:777]).max() < 3e-2
        finally:
            opc.SPMM_BLOCK_COST[variant], opc.SPMM_LONG_ROW[variant] = saved
    # the two kernels agree up to the 2^-17 relative rounding of the tensor-core kernel's split weights
    base = opc.spmm(Ad, Hd, variant=3 - variant).float().cpu()
    assert ((out - base).abs() / scale).max() < 1e-2
    # run to run the result is bitwise the same (pieces are summed in index order)
    first = opc.spmm(Ad, Hd, variant=variant)
    again = opc.spmm(Ad, Hd, variant=variant)
    assert torch.equal(first, again)


def test_spmm_fp32_features_and_empty_matrix():
    from plexus_b200 import ops

    A = _random_csr(200, 100, 5, seed=2)
    H = torch.randn(100, 64)
    out = ops.spmm(A.to(_dev()), H.to(_dev()))
    ref = torch.sparse.mm(A, H)
    assert torch.allclose(out.cpu(), ref, rtol=1e-4, atol=1e-4)
    Z = torch.sparse_csr_tensor(torch.zeros(51, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                                torch.zeros(0), size=(50, 100))
    out = ops.spmm(Z.to(_dev()), H.to(_dev()))
    assert out.shape == (50, 64) and float(out.abs().max()) == 0.0


NT_SHAPES = [(1000, 104, 256), (4096, 256, 256), (333, 64, 24), (129, 608, 256), (777, 128, 512),
             (5000, 24, 128), (128, 8, 8), (100000, 256, 48)]


@pytest.mark.parametrize("M,K,N", NT_SHAPES)
@pytest.mark.parametrize("trans_b", [False, True])
def test_gemm_nt_tcgen05(M, K, N, trans_b):
    from plexus_b200 import ops
    from plexus_b200.ops import cuda as opc

    torch.manual_seed(M + K + N)
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(K, N) / K ** 0.5)
    wb = w.to(torch.bfloat16)
    ref = a.float() @ wb.float()
    if trans_b:
        out = ops.gemm(a.to(_dev()), wb.t().contiguous().to(_dev()), trans_b=True)
    else:
        out = ops.gemm(a.to(_dev()), wb.to(_dev()))
    opc.check_status()
    assert out.dtype == torch.bfloat16 and out.shape == (M, N)
    err = (out.float().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 1e-2, err


def test_gemm_nt_relu_fp32_out_and_variants():
    from plexus_b200.ops import cuda as opc

    torch.manual_seed(0)
    a = torch.randn(3000, 256).to(torch.bfloat16)
    w = (torch.randn(256, 128) / 16).to(torch.bfloat16)
    ref = torch.relu(a.float() @ w.float())
    for v in range(len(opc.GEMM_VARIANTS)):
        out = opc.gemm(a.to(_dev()), w.to(_dev()), relu=True, out_dtype=torch.float32, variant=v)
        opc.check_status()
        assert out.dtype == torch.float32
        assert (out.cpu() - ref).abs().max() / ref.abs().max() < 2e-3, v


TN_SHAPES = [(5000, 104, 256), (70000, 256, 256), (999, 24, 48), (3000, 608, 256), (64, 8, 8),
             (20000, 128, 24), (4097, 256, 512)]


@pytest.mark.parametrize("R,Mw,Nw", TN_SHAPES)
def test_gemm_tn_tcgen05(R, Mw, Nw):
    from plexus_b200 import ops
    from plexus_b200.ops import cuda as opc

    torch.manual_seed(R + Mw + Nw)
    a = torch.randn(R, Mw).to(torch.bfloat16)
    b = torch.randn(R, Nw).to(torch.bfloat16)
    ref = a.double().t() @ b.double()
    out = ops.gemm(a.to(_dev()), b.to(_dev()), trans_a=True, out_dtype=torch.float32)
    opc.check_status()
    assert out.dtype == torch.float32 and out.shape == (Mw, Nw)
    err = (out.double().cpu() - ref).abs().max() / ref.abs().max()
    assert err < 1e-3, err
    # deterministic split reduction: bitwise identical when repeated
    out2 = ops.gemm(a.to(_dev()), b.to(_dev()), trans_a=True, out_dtype=torch.float32)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("C,class_offset,num_classes", [(48, 0, 47), (24, 24, 47), (8, 40, 41), (64, 64, 70),
                                                        (172, 0, 172), (300, 0, 290), (5, 0, 5), (44, 44, 60)])
def test_xent_kernels(dtype, C, class_offset, num_classes):
    from plexus_b200.ops import cuda as opc, reference as ref

    torch.manual_seed(C)
    R, num_nodes, row_offset = 1003, 990, 0
    logits = (torch.randn(R, C) * 3).to(dtype)
    target = torch.randint(-1, num_classes, (R,))
    ld = logits.to(_dev())
    td = target.to(_dev())
    m, s = opc.xent_local_stats(ld, class_offset, num_classes)
    m_ref, s_ref = ref.xent_local_stats(logits, class_offset, num_classes)
    assert torch.allclose(m.cpu(), m_ref) and torch.allclose(s.cpu(), s_ref, rtol=1e-3)
    gmax = m_ref + 0.5
    gsum = s_ref * torch.exp(m_ref - gmax) + 1.0  # pretend other shards contribute
    loss = opc.xent_combine_loss(ld, td, gmax.to(_dev()), gsum.to(_dev()), row_offset, class_offset, num_nodes)
    loss_ref = ref.xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes)
    assert torch.allclose(loss.cpu(), loss_ref, rtol=2e-3)
    scale = torch.tensor(0.37 / num_nodes)
    g = opc.xent_grad(ld, td, gmax.to(_dev()), gsum.to(_dev()), row_offset, class_offset, num_nodes,
                      num_classes, scale.to(_dev()))
    g_ref = ref.xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, num_classes,
                          scale, out_dtype=torch.float32)
    assert g.dtype == dtype
    assert (g.float().cpu() - g_ref).abs().max() <= 1e-2 * g_ref.abs().max() + 1e-7
    # statistics and loss in one launch (classes not sharded), with row weights
    w = torch.rand(R)
    st, l1 = opc.xent_stats(ld, class_offset, num_classes, td, row_offset, num_nodes, w.to(_dev()))
    st_ref, l1_ref = ref.xent_stats(logits, class_offset, num_classes, target, row_offset, num_nodes, w)
    assert torch.allclose(st.cpu(), st_ref, rtol=1e-3) and torch.allclose(l1.cpu(), l1_ref, rtol=2e-3)
    # the combine kernel: three class shards' statistics (one of them empty: (-inf, 0)) -> global + loss
    pairs = torch.stack([st_ref, torch.stack([m_ref - 1.0, s_ref * 2]),
                         torch.stack([torch.full_like(m_ref, float("-inf")), torch.zeros_like(s_ref)])])
    st2, l2 = opc.xent_combine(ld, td, pairs.to(_dev()), row_offset, class_offset, num_nodes, w.to(_dev()))
    st2_ref, l2_ref = ref.xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, w)
    assert torch.allclose(st2.cpu(), st2_ref, rtol=1e-3) and torch.allclose(l2.cpu(), l2_ref, rtol=2e-3)
    # rows that are not 16-byte aligned (a column slice of a wider matrix) take the element path
    if C >= 8:
        wide = torch.zeros(R, C + 3, dtype=dtype, device=_dev())
        wide[:, 1 : C + 1] = ld
        st3, _ = opc.xent_stats(wide[:, 1 : C + 1], class_offset, num_classes)
        assert torch.allclose(st3.cpu(), st_ref, rtol=1e-3)


def test_adam_multi_matches_reference():
    from plexus_b200.ops import cuda as opc, reference as ref

    torch.manual_seed(0)
    shapes = [(1000,), (4097,), (33,), (70000,)]
    dts = [torch.float32, torch.bfloat16, torch.float32, torch.bfloat16]
    P = [torch.randn(s).to(d) for s, d in zip(shapes, dts)]
    Gs = [torch.randn(s).to(d) for s, d in zip(shapes, dts)]
    M = [torch.randn(s).abs() * 0.1 for s in shapes]
    V = [torch.randn(s).abs() * 0.1 for s in shapes]
    W = [p.float().clone() if p.dtype != torch.float32 else None for p in P]
    dev = _dev()
    Pd, Gd, Md, Vd = ([t.clone().to(dev) for t in L] for L in (P, Gs, M, V))
    Wd = [w.clone().to(dev) if w is not None else None for w in W]
    for step in (1, 2):
        ref.adam_step(P, Gs, M, V, W, step, 3e-3, 0.9, 0.999, 1e-8, 0.01, True)
        opc.adam_step(Pd, Gd, Md, Vd, Wd, step, 3e-3, 0.9, 0.999, 1e-8, 0.01, True)
    for a, b in zip(P, Pd):
        assert torch.allclose(a.float(), b.float().cpu(), rtol=1e-2 if a.dtype == torch.bfloat16 else 1e-5, atol=1e-5)
    for a, b in zip(M + V, Md + Vd):
        assert torch.allclose(a, b.cpu(), rtol=1e-5, atol=1e-7)
    for a, b in zip(W, Wd):
        if a is not None:
            assert torch.allclose(a, b.cpu(), rtol=1e-5, atol=1e-6)


def test_relu_backward_and_prep_weight():
    from plexus_b200.ops import _ext, cuda as opc

    for dt in (torch.bfloat16, torch.float32):
        g = torch.randn(1001, 24).to(dt)
        y = torch.randn(1001, 24).to(dt)
        out = opc.relu_backward(g.to(_dev()), y.to(_dev()))
        assert torch.equal(out.cpu(), g * (y > 0))
    W = torch.randn(104, 48)
    Wb = torch.empty(104, 48, dtype=torch.bfloat16, device=_dev())
    WbT = torch.empty(48, 104, dtype=torch.bfloat16, device=_dev())
    _ext.load().prep_weight(W.to(_dev()), Wb, WbT)
    assert torch.equal(Wb.cpu(), W.to(torch.bfloat16))
    assert torch.equal(WbT.cpu(), W.to(torch.bfloat16).t().contiguous())


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A wait on a flag nobody raises must end in a status word, not a hang."""
    from plexus_b200.ops import _ext
    from plexus_b200.parallel.watchdog import PlexusCommTimeout, raise_on_device_status

    flag = torch.zeros(1, dtype=torch.int32, device=_dev())
    status = torch.zeros(8, dtype=torch.int32, device=_dev())
    _ext.load().wait_flag(flag, 1, 2000, status)
    with pytest.raises(PlexusCommTimeout):
        raise_on_device_status(status)
    # the context is still usable and the status was cleared
    assert int(status[0]) == 0
    flag.fill_(1)
    _ext.load().wait_flag(flag, 1, 2000, status)
    raise_on_device_status(status)


def test_startup_kernels_match_the_torch_versions():
    from plexus_b200.data import graph_ops, synthetic

    dev = _dev()
    # R-MAT stream: device kernel == torch integer arithmetic on the CPU
    r_gpu, c_gpu = synthetic.rmat_edges(100000, 12345, 50000, seed=9, device=dev)
    r_cpu, c_cpu = synthetic.rmat_edges(100000, 12345, 50000, seed=9, device="cpu")
    assert torch.equal(r_gpu.cpu(), r_cpu) and torch.equal(c_gpu.cpu(), c_cpu)
    # whole synthetic graph identical on both devices
    d_gpu, _ = synthetic.synthetic_graph(3000, 20000, 8, 4, seed=2, device=dev)
    d_cpu, _ = synthetic.synthetic_graph(3000, 20000, 8, 4, seed=2, device="cpu")
    assert torch.equal(d_gpu.edge_index.cpu(), d_cpu.edge_index)
    assert torch.allclose(d_gpu.edge_weight.cpu(), d_cpu.edge_weight, rtol=1e-5)
    assert torch.allclose(d_gpu.x.cpu(), d_cpu.x, atol=1e-5) and torch.equal(d_gpu.y.cpu(), d_cpu.y)
    # COO -> CSR with shuffled input
    g = torch.Generator().manual_seed(0)
    rows, cols = 500, 700
    key = torch.unique(torch.randint(0, rows * cols, (6000,), generator=g))
    key = key[torch.randperm(key.numel(), generator=g)]
    row, col, val = key // cols, key % cols, torch.rand(key.numel(), generator=g)
    want = graph_ops.coo_to_csr(row, col, val, rows, cols)
    got = graph_ops.coo_to_csr(row.to(dev), col.to(dev), val.to(dev), rows, cols)
    for a, b in zip(got, want):
        assert a.dtype == b.dtype and torch.equal(a.cpu(), b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_relu_dropout_same_mask_on_cpu_and_gpu(dtype):
    from plexus_b200.ops.dropout import relu_dropout

    torch.manual_seed(0)
    x = torch.randn(1000, 24).to(dtype)
    g = torch.randn(1000, 24).to(dtype)
    outs = []
    for dev in ("cpu", _dev()):
        xi = x.detach().clone().to(dev).requires_grad_()
        y = relu_dropout(xi, p=0.3, seed=5, index_offset=77)
        y.backward(g.to(dev))
        outs.append((y.detach().float().cpu(), xi.grad.float().cpu()))
    assert torch.allclose(outs[0][0], outs[1][0], rtol=1e-2, atol=1e-3)
    assert torch.allclose(outs[0][1], outs[1][1], rtol=1e-2, atol=1e-3)
    kept = (outs[1][0] != 0).float().sum() / (x > 0).float().sum()
    assert 0.6 < kept < 0.8
    y0 = relu_dropout(x.to(_dev()), p=0.0)
    assert torch.equal(y0.cpu(), torch.relu(x))


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_nt_relu_derivative_mask_in_epilogue(out_dtype):
    from plexus_b200.ops import cuda as opc

    torch.manual_seed(3)
    a = torch.randn(1111, 48).to(torch.bfloat16)
    w = (torch.randn(256, 48) / 7).to(torch.bfloat16)  # [N, K]: used transposed
    mask = torch.randn(1111, 256).to(out_dtype)
    mask[::5] = 0
    ref = (a.float() @ w.float().t()) * (mask.float() > 0)
    out = opc.gemm(a.to(_dev()), w.to(_dev()), trans_b=True, out_dtype=out_dtype, relu_mask=mask.to(_dev()))
    opc.check_status()
    assert out.dtype == out_dtype
    assert (out.float().cpu() - ref).abs().max() < 1e-2 * ref.abs().max()
    assert torch.equal(out.float().cpu() == 0, ref == 0)


def test_csr_validate_reports_bad_structure_without_touching_memory_through_it():
    """The validator reads only the index arrays themselves; a bad index ends in a status word."""
    from plexus_b200.ops import cuda as opc

    A = _random_csr(500, 300, 6.0, seed=4).to(_dev())
    opc.validate_csr(A)  # a well-formed matrix passes
    crow, col, val = A.crow_indices().clone(), A.col_indices().clone(), A.values()
    bad_col = col.clone()
    bad_col[17] = 300  # one past the last column
    B = torch.sparse_csr_tensor(crow, bad_col, val, size=(500, 300), check_invariants=False)
    with pytest.raises(RuntimeError, match="csr_validate"):
        opc.validate_csr(B)
    bad_crow = crow.clone()
    bad_crow[200] = bad_crow[201] + 1  # not monotone
    Cm = torch.sparse_csr_tensor(bad_crow, col, val, size=(500, 300), check_invariants=False)
    with pytest.raises(RuntimeError, match="csr_validate"):
        opc.validate_csr(Cm)
    opc.validate_csr(A)  # the status was cleared, the context is fine
    # host-side shape checks of the SpMM wrapper
    with pytest.raises(ValueError):
        opc.spmm(A, torch.zeros(299, 8, dtype=torch.bfloat16, device=_dev()))


def test_weight_shard_kernel_equals_the_host_hash():
    from plexus_b200.models.gcn_conv import init_full_weight, init_weight_shard

    in_ch, out_ch, layer, seed = 100, 47, 1, 3
    full = torch.nn.functional.pad(init_full_weight(in_ch, out_ch, layer, seed), (0, 1, 0, 4))  # 104 x 48
    lr, lc = 52, 24
    for i in range(2):
        for o in range(2):
            block = full[i * lr:(i + 1) * lr, o * lc:(o + 1) * lc].reshape(-1)
            for d in range(2):
                per = block.numel() // 2
                got = init_weight_shard(in_ch, out_ch, layer, seed, i * lr, o * lc, lc, d * per, per, _dev())
                assert torch.equal(got.cpu(), block[d * per:(d + 1) * per]), (i, o, d)


def test_position_keyed_dropout_mask_is_the_same_on_cpu_and_gpu():
    from plexus_b200.ops.dropout import keep_mask_2d, relu_dropout_2d

    a = keep_mask_2d(300, 40, 0.25, 9, 1000, 8, 64)
    b = keep_mask_2d(300, 40, 0.25, 9, 1000, 8, 64, device=_dev())
    assert torch.equal(a, b.cpu()) and 0.6 < a.float().mean() < 0.9
    x = torch.randn(300, 40).to(torch.bfloat16)
    y_cpu = relu_dropout_2d(x, 0.25, 9, 1000, 8, 64)
    xg = x.to(_dev()).requires_grad_()
    y_gpu = relu_dropout_2d(xg, 0.25, 9, 1000, 8, 64)
    assert torch.equal(y_cpu, y_gpu.detach().cpu())
    y_gpu.float().sum().backward()
    want = ((y_cpu > 0).float() / 0.75).to(torch.bfloat16)
    assert torch.equal(xg.grad.cpu(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("op", ["gemm", "spmm"])
def test_debug_bounds_check_of_the_push_stores(op):
    """With a slot capacity attached to the push targets (what PLEXUS_DEBUG=1 does) a store that would
    end beyond the receive slot is skipped and recorded in the status words; nothing faults.  A local
    buffer stands in for the peer's slot."""
    from plexus_b200.data import graph_ops
    from plexus_b200.ops import cuda as opc
    from plexus_b200.parallel.symm import PushList

    torch.manual_seed(3)
    rows, K, N = 384, 64, 64
    slot = torch.full((rows, N), -1.0, dtype=torch.bfloat16, device=_dev())
    targets = PushList([slot.data_ptr()])
    targets.limit_bytes = rows // 2 * N * 2  # the slot "ends" after half of the rows
    if op == "gemm":
        a = torch.randn(rows, K).to(torch.bfloat16).to(_dev())
        w = (torch.randn(K, N) / 8).to(torch.bfloat16).to(_dev())
        out = opc.gemm(a, w, push_ptrs=targets, push_ld=N)
    else:
        dense = (torch.rand(rows, 200) < 0.05).float() * torch.randn(rows, 200)
        sp = dense.to_sparse_coo().coalesce()
        crow, col, val = graph_ops.coo_to_csr(sp.indices()[0].to(_dev()), sp.indices()[1].to(_dev()),
                                              sp.values().to(_dev()), rows, 200)
        A = graph_ops.csr_tensor(crow, col, val, (rows, 200))
        H = torch.randn(200, N).to(torch.bfloat16).to(_dev())
        out = opc.spmm(A, H, push_ptrs=targets, push_ld=N)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="BOUNDS"):
        opc.check_status()
    assert torch.equal(slot[: rows // 2], out[: rows // 2])           # stores inside the slot went through
    assert bool((slot[rows // 2 :] == -1).all())                      # the others were skipped
    opc.check_status()                                                # the record was cleared
    # with the whole slot as capacity nothing is reported
    targets.limit_bytes = rows * N * 2
    if op == "gemm":
        out = opc.gemm(a, w, push_ptrs=targets, push_ld=N)
    else:
        out = opc.spmm(A, H, push_ptrs=targets, push_ld=N)
    opc.check_status()
    assert torch.equal(slot, out)


@pytest.mark.gpu
def test_offsets_beyond_two_gib_through_large_row_pitches():
    """Element offsets above 2^31 bytes in H, the output and the GEMM operands (what a 55M-row shard
    produces), reached with few rows by giving the matrices a row pitch of 1 MB."""
    from plexus_b200.data import graph_ops
    from plexus_b200.ops import cuda as opc

    free, _ = torch.cuda.mem_get_info()
    if free < 16 << 30:
        pytest.skip("needs 16 GB of free device memory")
    torch.manual_seed(11)
    rows, cols, D, pitch = 2600, 3000, 64, 512 * 1024  # (cols - 1) * pitch * 2 bytes = 3.1 GB
    dense = (torch.rand(rows, cols) < 0.01).float() * torch.randn(rows, cols)
    dense[5, :] = torch.randn(cols)  # one long row (pieces)
    sp = dense.to_sparse_coo().coalesce()
    crow, col, val = graph_ops.coo_to_csr(sp.indices()[0].to(_dev()), sp.indices()[1].to(_dev()),
                                          sp.values().to(_dev()), rows, cols)
    A = graph_ops.csr_tensor(crow, col, val, (rows, cols))
    Hs = torch.randn(cols, D).to(torch.bfloat16)
    Hbig = torch.zeros(cols, pitch, dtype=torch.bfloat16, device=_dev())
    Hbig[:, :D] = Hs.to(_dev())
    obig = torch.zeros(rows, pitch, dtype=torch.bfloat16, device=_dev())
    want = dense @ Hs.float()
    for variant in (1, 2):
        obig[:, :D].zero_()
        out = opc.spmm(A, Hbig[:, :D], out=obig[:, :D], variant=variant)
        assert out.data_ptr() == obig.data_ptr()
        err = (out.float().cpu() - want).abs().max().item()
        assert err <= 1e-2 * want.abs().max().item(), (variant, err)
    assert bool((obig[:, D : D + 64] == 0).all())  # nothing written beside the D columns
    # GEMM reading A and writing C with the same pitch; the last rows lie beyond 2^31 bytes
    W = (torch.randn(D, 128) / 8).to(torch.bfloat16)
    cbig = torch.zeros(rows, pitch, dtype=torch.bfloat16, device=_dev())
    got = opc.gemm(obig[:, :D], W.to(_dev()), out=cbig[:, :128])
    ref = obig[:, :D].float().cpu() @ W.float()
    assert (got.float().cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    # weight gradient (split-K over the rows) from the same strided operands
    gw = opc.gemm(obig[:, :D], cbig[:, :128], trans_a=True, out_dtype=torch.float32)
    refw = obig[:, :D].float().cpu().t() @ cbig[:, :128].float().cpu()
    assert (gw.cpu() - refw).abs().max().item() <= 2e-2 * refw.abs().max().item()
    opc.check_status()


@pytest.mark.gpu
def test_xent_statistics_pushed_into_receive_slots_and_combined_by_address():
    """The exchange forms of the cross-entropy kernels on one GPU: local buffers stand in for the peers'
    receive slots (no flags: the combine kernel's barrier is off when no flag lists are given)."""
    from plexus_b200.ops import cuda as opc, reference as ref

    torch.manual_seed(21)
    R, C, num_classes, num_nodes = 3001, 24, 47, 2990
    shards = [(torch.randn(R, C) * 2).to(torch.bfloat16) for _ in range(2)]  # class shards 0 and 1
    target = torch.randint(-1, num_classes, (R,))
    slots = [torch.full((2, R), float("nan"), device=_dev()) for _ in range(2)]  # "peer" slots for shard 1's pairs
    st1, _ = opc.xent_stats(shards[1].to(_dev()), C, num_classes, push_ptrs=[s.data_ptr() for s in slots])
    torch.cuda.synchronize()
    st1_ref, _ = ref.xent_stats(shards[1], C, num_classes)
    assert torch.allclose(st1.cpu(), st1_ref, rtol=1e-3)
    assert all(torch.equal(s, st1) for s in slots)  # the pushed pairs are the local ones, bit for bit
    # rank 0's combine: own statistics by address + shard 1's pairs from the "receive slot"
    st0, _ = opc.xent_stats(shards[0].to(_dev()), 0, num_classes)
    stats, loss = opc.xent_combine_ptrs(shards[0].to(_dev()), target.to(_dev()), [st0.data_ptr(), slots[0].data_ptr()],
                                        0, 0, num_nodes)
    st0_ref, _ = ref.xent_stats(shards[0], 0, num_classes)
    stats_ref, loss_ref = ref.xent_combine(shards[0], target, torch.stack([st0_ref, st1_ref]), 0, 0, num_nodes)
    assert torch.allclose(stats.cpu(), stats_ref, rtol=1e-3) and torch.allclose(loss.cpu(), loss_ref, rtol=2e-3)
    opc.check_status()
