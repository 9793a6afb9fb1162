"""Per-rank bodies of the multi-process tests (must be importable for spawn)."""
import torch
import torch.distributed as dist


def _inputs(rank, m_rows, n, k, dtype, seed=1234):
    # seeded on the CPU so that the CPU oracle and the GPU op see identical values
    g = torch.Generator().manual_seed(seed + rank)
    a = torch.randn(m_rows, k, generator=g).to(dtype)
    b = (torch.randn(n, k, generator=g) * 0.02).to(dtype)
    return a, b


def ag_gemm_case(rank, world, shapes, dtype_name, with_bias, tuning):
    """AGKernel.forward vs the gloo golden path, several calls on one op (ragged M, both parities)."""
    import flux_b200 as flux
    from oracle import golden

    dtype = getattr(torch, dtype_name)
    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    full_m = max(s[0] for s in shapes) * world
    n_dim = max(s[1] for s in shapes)
    k = shapes[0][2]
    op = flux.AGKernel(group, 1, full_m, n_dim, k, dtype)
    for it, (m_local, n, kk) in enumerate(shapes):
        assert kk == k
        a, b = _inputs(rank, m_local, n, k, dtype, seed=1234 + 17 * it)
        bias = None
        if with_bias:
            g = torch.Generator().manual_seed(99 + rank + it)
            bias = (torch.randn(m_local * world, n, generator=g) * 0.1).to(dtype)
        ref, ref_gathered = golden.ag_gemm_dist(group, a, b, bias)
        gathered = torch.empty((m_local * world, k), dtype=dtype, device="cuda")
        out = op.forward(a.cuda(), b.cuda(), bias=None if bias is None else bias.cuda(),
                         gathered_input=gathered, tuning=tuning)
        torch.cuda.synchronize()
        comm.check_status()
        # tolerance: max relative error <= 1e-2 for 16-bit inputs with fp32 accumulation
        err = golden.max_rel_err(out, ref)
        assert err <= 1e-2, f"rank {rank} call {it} shape {(m_local, n, k)}: max rel err {err}"
        assert torch.equal(gathered.cpu().view(torch.int16), ref_gathered.view(torch.int16)), \
            f"rank {rank} call {it}: gathered input differs from all_gather"


def gemm_rs_case(rank, world, shapes, dtype_name, with_bias, tuning, fp32_wire=False):
    """GemmRS.forward vs the gloo golden path, several calls on one op."""
    import flux_b200 as flux
    from oracle import golden

    dtype = getattr(torch, dtype_name)
    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    max_m = max(s[0] for s in shapes)
    n = shapes[0][1]
    op = flux.GemmRS(group, 1, max_m, n, dtype)
    op.fp32_wire = fp32_wire
    for it, (m, nn, k_local) in enumerate(shapes):
        assert nn == n
        a, b = _inputs(rank, m, n, k_local, dtype, seed=4321 + 17 * it)
        bias = None
        if with_bias:
            g = torch.Generator().manual_seed(77 + rank + it)
            bias = (torch.randn(m, n, generator=g) * 0.1).to(dtype)
        # golden: fp32 partials over gloo (the reference and the product's default reduce partials that were
        # rounded to the output format; fp32_wire keeps them fp32)
        part = golden._rs_partial(a, b, bias, None, None).float().contiguous()
        dist.all_reduce(part, group=group)
        mpr = m // world
        ref = part[rank * mpr:(rank + 1) * mpr]
        out = op.forward(a.cuda(), b.cuda(), bias=None if bias is None else bias.cuda(), tuning=tuning)
        torch.cuda.synchronize()
        comm.check_status()
        err = golden.max_rel_err(out, ref)
        assert err <= 1e-2, f"rank {rank} call {it} shape {(m, n, k_local)}: max rel err {err}"


def moe_case(rank, world, cfgs, dtype_name):
    """MoE layer 0 (AG + scatter + grouped GEMM) and layer 1 (grouped GEMM + gather + RS) vs the gloo oracle."""
    import flux_b200 as flux
    from oracle import golden

    dtype = getattr(torch, dtype_name)
    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    for ci, (ntokens, topk, nexperts, hidden, ffn, calls) in enumerate(cfgs):
        ffn_local = ffn // world
        env = flux.DistEnvTPWithEP(group, 1, None)
        margs = flux.MoeArguments(ntokens, hidden, ffn, nexperts, topk, dtype)
        l0 = flux.GemmGroupedV3AGScatter(env, margs)
        l1 = flux.GemmGroupedV3GatherRS(nexperts, ntokens * topk, hidden, topk, rank, world, world, 1, input_dtype=dtype)
        for it in range(calls):
            g = torch.Generator().manual_seed(1234 + 31 * ci + it)  # routing is global: same seed on every rank
            logits = torch.randn(ntokens, nexperts, generator=g)
            if it == 1:
                logits[:, 0] = -1e9  # an expert that receives no tokens
            chosen, rw = golden.topk_routing(logits, topk)
            si = golden.calc_scatter_index_stable(chosen)
            splits = golden.calc_splits(chosen, nexperts)
            gi, ti = golden.calc_gather_index(si)
            gr = torch.Generator().manual_seed(999 + rank + 7 * it)
            tok = torch.randn(ntokens // world, hidden, generator=gr).to(dtype)
            w0 = (torch.randn(nexperts, ffn_local, hidden, generator=gr) * 0.02).to(dtype)
            w1 = (torch.randn(nexperts, hidden, ffn_local, generator=gr) * 0.02).to(dtype)
            oscale = torch.rand(nexperts, generator=gr) + 0.5
            # ---- layer 0
            shards = [torch.empty_like(tok) for _ in range(world)]
            dist.all_gather(shards, tok, group=group)
            ref0, ref_g = golden.moe_ag_scatter_single(shards, w0, splits, si, oscale)
            gathered = torch.empty((ntokens, hidden), dtype=dtype, device="cuda")
            out0 = l0.forward(tok.cuda(), w0.cuda(), splits.cuda(), si.cuda(), output_scale=oscale.cuda(),
                              allgather_output=gathered)
            torch.cuda.synchronize()
            comm.check_status()
            err0 = golden.max_rel_err(out0, ref0)
            assert err0 <= 1e-2, f"rank {rank} cfg {ci} call {it}: layer 0 max rel err {err0}"
            assert torch.equal(gathered.cpu().view(torch.int16), ref_g.view(torch.int16))
            # ---- layer 1 (input = the oracle's layer-0 output so that errors do not compound)
            vec = rw.reshape(-1)[(gi.long() * topk + ti.long())].contiguous()
            ref1 = golden.moe_gather_rs_dist(group, ref0, w1, splits, si, topk, output_vec_scale=vec)
            out1 = l1.forward_gather_rs(ref0.cuda(), w1.cuda(), splits, si.reshape(-1).cuda(), output_vec_scale=vec.cuda())
            torch.cuda.synchronize()
            comm.check_status()
            # tolerance of the reference's own test for bf16 (test_moe_gather_rs.py:397-411): 2e-2
            err1 = golden.max_rel_err(out1, ref1)
            assert err1 <= 2e-2, f"rank {rank} cfg {ci} call {it}: layer 1 max rel err {err1}"


def fp8_case(rank, world, shapes):
    """FP8 e4m3 AG-GEMM with per-row input scales (all-gathered by the op) and per-channel weight scales,
    and FP8 GEMM-RS, against the dequantised oracle (tolerance 3e-2)."""
    import flux_b200 as flux
    from oracle import golden

    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    f8 = torch.float8_e4m3fn
    for it, (m_local, n, k) in enumerate(shapes):
        g = torch.Generator().manual_seed(555 + rank + 13 * it)
        a = torch.randn(m_local, k, generator=g)
        b = torch.randn(n, k, generator=g) * 0.02
        qa, sa = golden.quantize_fp8_rows(a)
        qb, sb = golden.quantize_fp8_rows(b)
        ref, _ = golden.ag_gemm_dist(group, qa, qb, None, sa, sb)
        op = flux.AGKernel(group, 1, m_local * world, n, k, f8)
        out = op.forward(qa.cuda(), qb.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda())
        torch.cuda.synchronize()
        comm.check_status()
        assert out.dtype == torch.bfloat16
        err = golden.max_rel_err(out, ref)
        assert err <= 3e-2, f"rank {rank} call {it}: fp8 AG-GEMM max rel err {err}"
        # GEMM-RS: A [M, k] fp8 with per-row scale, B [n, k] fp8 with per-channel scale
        m = m_local * world
        a2 = torch.randn(m, k, generator=g)
        qa2, sa2 = golden.quantize_fp8_rows(a2)
        part = golden._rs_partial(qa2, qb, None, sa2, sb).float().contiguous()
        dist.all_reduce(part, group=group)
        mpr = m // world
        rs = flux.GemmRS(group, 1, m, n, f8)
        out2 = rs.forward(qa2.cuda(), qb.cuda(), input_scale=sa2.cuda(), weight_scale=sb.cuda())
        torch.cuda.synchronize()
        comm.check_status()
        err2 = golden.max_rel_err(out2, part[rank * mpr:(rank + 1) * mpr])
        assert err2 <= 3e-2, f"rank {rank} call {it}: fp8 GEMM-RS max rel err {err2}"


def tp_mlp_case(rank, world):
    """TensorParallelMLP forward + backward on `world` GPUs against the unsharded fp32 model (gloo gathers)."""
    import flux_b200 as flux

    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    hidden, ffn, tokens = 512, 256 * world, 128 * world
    torch.manual_seed(21 + rank)
    mlp = flux.TensorParallelMLP(hidden, ffn, tokens, group)
    x_shard = torch.randn(tokens // world, hidden, device="cuda").bfloat16().requires_grad_(True)
    g_shard = torch.randn(tokens // world, hidden, device="cuda").bfloat16()
    y_shard = mlp(x_shard)
    (y_shard.float() * g_shard.float()).sum().backward()
    torch.cuda.synchronize()
    comm.check_status()

    def gather(t, dim):
        parts = [torch.empty_like(t.cpu()) for _ in range(world)]
        dist.all_gather(parts, t.detach().cpu().contiguous(), group=group)
        return torch.cat(parts, dim=dim).float()

    w1 = gather(mlp.fc1.weight, 0).requires_grad_(True)
    w2 = gather(mlp.fc2.weight, 1).requires_grad_(True)
    x = gather(x_shard, 0).requires_grad_(True)
    g = gather(g_shard, 0)
    y = torch.nn.functional.gelu((x @ w1.t()).bfloat16().float()) @ w2.t()
    (y * g).sum().backward()
    mpr, fl = tokens // world, ffn // world
    rows, cols = slice(rank * mpr, (rank + 1) * mpr), slice(rank * fl, (rank + 1) * fl)

    def rel(a, b):
        return float((a.float().cpu() - b).abs().max() / b.abs().max())

    assert rel(y_shard, y.detach()[rows]) <= 2e-2
    assert rel(x_shard.grad, x.grad[rows]) <= 2e-2
    assert rel(mlp.fc1.weight.grad, w1.grad[cols]) <= 2e-2
    assert rel(mlp.fc2.weight.grad, w2.grad[:, cols]) <= 2e-2


def baseline_shapes_case(rank, world):
    """The dense BASELINE configurations at this world size, one process per GPU: D0 (AG-GEMM M=4096, N=49152/TP,
    K=12288) feeding D1 (GEMM-RS M=4096, N=12288, K=49152/TP), both all-gather transports, and F (fp8 AG-GEMM
    M=8192, N=28672/TP, K=8192 with per-row x per-channel scales); checked by fp64 dot products on sampled entries,
    rows of every source rank included (the CPU oracle would take minutes at these sizes)."""
    import flux_b200 as flux

    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    M, N0, K0, N1 = 4096, 49152, 12288, 12288
    m_local, n_local = M // world, N0 // world
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    a = torch.randn(m_local, K0, generator=g, device="cuda").bfloat16()
    b0 = (torch.randn(n_local, K0, generator=g, device="cuda") * 0.02).bfloat16()
    b1 = (torch.randn(N1, n_local, generator=g, device="cuda") * 0.02).bfloat16()

    def spread(n, count):
        return torch.tensor([round(i * (n - 1) / (count - 1)) for i in range(count)], device="cuda")

    def all_gather_cuda(x):
        # the spawn helper runs over gloo: gather through the host
        host = [torch.empty_like(x.cpu()) for _ in range(world)]
        dist.all_gather(host, x.cpu().contiguous(), group=group)
        return torch.cat(host).cuda()

    def all_reduce_cuda(x):
        h = x.cpu()
        dist.all_reduce(h, group=group)
        return h.cuda()

    def check(got, exact, tol_rel, tol_elem, what):
        got, exact = got.double(), exact.double()
        rel = float((got - exact).abs().max() / exact.abs().max())
        assert rel <= tol_rel, f"rank {rank} {what}: max rel err {rel}"
        assert bool(((got - exact).abs() <= tol_elem + tol_elem * exact.abs()).all()), f"rank {rank} {what}: elementwise {tol_elem}"

    ag = flux.AGKernel(group, 1, M, n_local, K0, torch.bfloat16)
    rs = flux.GemmRS(group, 1, M, N1, torch.bfloat16)
    rows_l, cols0, cols1 = spread(m_local, 8), spread(n_local, 16), spread(N1, 16)
    grows = (torch.arange(world, device="cuda")[:, None] * m_local + rows_l[None, :]).reshape(-1)
    a_rows = all_gather_cuda(a[rows_l]).double()
    exact0 = a_rows @ b0[cols0].double().t()
    for ag_mode in (1, 2):
        c0 = ag.forward(a, b0, tuning={"ag_mode": ag_mode})
        torch.cuda.synchronize()
        comm.check_status()
        check(c0[grows][:, cols0], exact0, 1e-2, 1e-2, f"D0 (all-gather transport {ag_mode})")
    out = rs.forward(c0, b1)
    torch.cuda.synchronize()
    comm.check_status()
    part = c0[grows].double() @ b1[cols1].double().t()
    exact1 = all_reduce_cuda(part)
    gold1 = all_reduce_cuda(part.bfloat16().double()).bfloat16()  # the golden path rounds every rank's partial to bf16
    lo = rank * rows_l.numel()
    got1 = out[rows_l][:, cols1]
    rel = float((got1.double() - exact1[lo:lo + rows_l.numel()]).abs().max() / exact1.abs().max())
    assert rel <= 1e-2, f"rank {rank} D1: max rel err vs fp64 {rel}"
    check(got1, gold1[lo:lo + rows_l.numel()], 1e-2, 2e-2, "D1 vs the golden path")
    del ag, rs, b0, b1, c0
    # ---- F: fp8 with per-row / per-channel scales
    f8 = torch.float8_e4m3fn
    FM, FN, FK = 8192, 28672, 8192
    fm, fn = FM // world, FN // world
    x = torch.randn(fm, FK, generator=g, device="cuda")
    w = torch.randn(fn, FK, generator=g, device="cuda") * 0.02
    sx = (x.abs().amax(1).clamp_min(1e-12) / 448.0).float()
    sw = (w.abs().amax(1).clamp_min(1e-12) / 448.0).float()
    qx, qw = (x / sx[:, None]).to(f8), (w / sw[:, None]).to(f8)
    op = flux.AGKernel(group, 1, FM, fn, FK, f8)
    o8 = op.forward(qx, qw, input_scale=sx, weight_scale=sw)
    torch.cuda.synchronize()
    comm.check_status()
    r8, c8 = spread(fm, 8), spread(fn, 16)
    g8 = (torch.arange(world, device="cuda")[:, None] * fm + r8[None, :]).reshape(-1)
    xr = all_gather_cuda(qx[r8].double() * sx[r8].double()[:, None])
    check(o8[g8][:, c8], xr @ (qw[c8].double() * sw[c8].double()[:, None]).t(), 3e-2, 3e-2, "F")


def runtime_case(rank, world):
    """Symmetric tensor list and the stream barrier across processes (reference test:
    test/python/util/test_flux_ring_barrier.py; src/ths_op/flux_shm.cc:434-452,656-733): every rank writes its own
    block, a barrier on the stream orders the writes, then every rank reads all peers' blocks through the mapped
    pointers and writes into the next peer's block."""
    import flux_b200 as flux

    group = dist.group.WORLD
    flux.init_flux_shm(group)
    comm = flux.get_comm(group)
    comm.set_timeout_ms(5000)
    ts = flux.flux_create_tensor_list((4, 64), torch.float32, group)
    assert len(ts) == world and all(t.shape == (4, 64) for t in ts)
    gb = flux.GroupBarrier(group)
    for it in range(3):
        ts[rank].fill_(float(10 * it + rank + 1))
        gb.barrier_all()
        for r in range(world):
            # peers' blocks are only ever touched by copies (copy engines), never handed to a library kernel
            got = ts[r].cpu()
            assert float(got.sum()) == 4 * 64 * (10 * it + r + 1), f"rank {rank} reads rank {r}'s block (iteration {it})"
        gb.barrier_all()  # nobody overwrites a block that a peer is still reading
    nxt = (rank + 1) % world
    ts[nxt][0].copy_(torch.full((64,), -float(rank + 1), device="cuda"))  # a copy into a peer's memory
    gb.barrier_all()
    torch.cuda.synchronize()
    prev = (rank - 1) % world
    assert float(ts[rank][0, 0]) == -float(prev + 1) and float(ts[rank][1, 0]) == 20.0 + rank + 1
    comm.check_status()
