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


def gemm_rs_case(rank, world, shapes, dtype_name, with_bias, tuning):
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
    for it, (m, nn, k_local) in enumerate(shapes):
        assert nn == n
        a, b = _inputs(rank, m, n, k_local, dtype, seed=4321 + 17 * it)
        bias = None
        if with_bias:
            g = torch.Generator().manual_seed(77 + rank + it)
            bias = (torch.randn(m, n, generator=g) * 0.1).to(dtype)
        # golden: fp32 partials over gloo (the reference reduces the rounded partials; the product keeps fp32)
        part = golden._rs_partial(a, b, bias, None, None).float().contiguous()
        dist.all_reduce(part, group=group)
        mpr = m // world
        ref = part[rank * mpr:(rank + 1) * mpr]
        out = op.forward(a.cuda(), b.cuda(), bias=None if bias is None else bias.cuda(), tuning=tuning)
        torch.cuda.synchronize()
        comm.check_status()
        err = golden.max_rel_err(out, ref)
        assert err <= 1e-2, f"rank {rank} call {it} shape {(m, n, k_local)}: max rel err {err}"
