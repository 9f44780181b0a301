"""Expert-parallel dispatch/combine against a plain PyTorch statement of the same routing.

Follows the reference's examples/device/ep/tests/elastic/elastic.py (correctness of dispatch
layout, fp8 cast, combine reduction; a silent rank is masked after a timeout instead of
hanging).  Ranks are Buffer objects of one process placed on different GPUs; cases that need
peers waiting on each other are skipped when only one GPU is present."""
import pytest
import torch

from nixl_b200.parallel import Buffer, dequant_fp8, dequant_ue8m0, per_token_cast_to_fp8

pytestmark = pytest.mark.gpu


def _make_ranks(n, experts, hidden, tokens, topk, timeout_ms=20000, tag="ep", **kw):
    from nixl_b200 import nixl_agent, nixl_agent_config

    bufs = []
    for r in range(n):
        dev = torch.device("cuda", r % torch.cuda.device_count())
        agent = nixl_agent(f"{tag}_rank{r}", nixl_agent_config(enable_prog_thread=False, backends=["NVLINK"]))
        with torch.cuda.device(dev):
            bufs.append(Buffer(r, n, experts, hidden, tokens, topk, device=dev, agent=agent, timeout_ms=timeout_ms, **kw))
    md = [b.local_metadata() for b in bufs]
    for b in bufs:
        b.connect_ranks(metadata=md)
    return bufs


def _inputs(bufs, tokens, hidden, experts, topk, seed=0):
    xs, idxs, ws = [], [], []
    for b in bufs:
        g = torch.Generator(device=b.device).manual_seed(seed + b.rank)
        x = torch.randn(tokens, hidden, device=b.device, dtype=torch.bfloat16, generator=g)
        logits = torch.randn(tokens, experts, device=b.device, generator=g)
        w, idx = torch.topk(torch.softmax(logits, dim=-1), topk, dim=-1)
        idx = idx.to(torch.int64).contiguous()
        idx[0, -1] = -1  # an unused slot must be skipped
        xs.append(x)
        idxs.append(idx)
        ws.append(w.float().contiguous())
    return xs, idxs, ws


def _check_dispatch(bufs, xs, idxs, results, use_fp8, compact):
    n, El = len(bufs), bufs[0].local_experts
    quant = [per_token_cast_to_fp8(x) if use_fp8 else (x, None) for x in xs]
    for d, b in enumerate(bufs):
        recv_x, scales, handle = results[d]
        counts = handle.recv_count.cpu()
        offs = handle.expert_offsets.cpu()
        info = handle.src_info.cpu()
        ranges = handle.layout_range.cpu()
        for le in range(El):
            e = d * El + le
            expect = sum(int((idxs[r] == e).sum()) for r in range(n))
            assert int(counts[le]) == expect, (d, le)
            start = int(offs[le])
            prev_rank, seen = -1, set()
            for j in range(expect):
                src, tk = int(info[start + j, 0]), int(info[start + j, 1])
                assert src >= prev_rank  # rows of an expert are ordered by source rank
                prev_rank = src
                t, k = divmod(tk, bufs[0].topk)
                assert int(idxs[src][t, k]) == e and (src, tk) not in seen
                seen.add((src, tk))
                got = recv_x[start + j].to(xs[src].device)
                if use_fp8:
                    # Same scale; codes may differ by one step where x * (448 / amax) lands on a
                    # rounding boundary (the division is rounded differently by the two programs).
                    torch.testing.assert_close(scales[start + j].to(xs[src].device), quant[src][1][t], rtol=1e-6, atol=0)
                    a = got.view(torch.uint8).to(torch.int16)
                    w = quant[src][0][t].view(torch.uint8).to(torch.int16)
                    diff = (a - w).abs()
                    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 0.02
                else:
                    assert torch.equal(got, xs[src][t])
            for r in range(n):
                first, rows = int(ranges[le, r]) >> 32, int(ranges[le, r]) & 0xFFFFFFFF
                assert rows == int((idxs[r] == e).sum())
                assert all(int(info[start + first + j, 0]) == r for j in range(rows))


def _run(bufs, tokens, hidden, experts, topk, use_fp8, compact, zero_copy=False, rank_reduce=False):
    xs, idxs, ws = _inputs(bufs, tokens, hidden, experts, topk)
    results = []
    for b, x, idx, w in zip(bufs, xs, idxs, ws):  # launch every rank before waiting on any
        with torch.cuda.device(b.device):
            if compact:
                results.append(b.dispatch(x, idx, use_fp8=use_fp8, topk_weights=w if rank_reduce else None))
                assert results[-1][2].has_group_records == rank_reduce
            else:
                recv, cnt, handle, _, _ = b.low_latency_dispatch(x, idx, use_fp8=use_fp8)
                El, rows = b.local_experts, b.num_ranks * b.max_tokens
                rx, sc = (recv if use_fp8 else (recv, None))
                results.append((rx.view(El * rows, hidden), sc.view(El * rows, -1) if sc is not None else None, handle))
    for b in bufs:
        torch.cuda.synchronize(b.device)
        assert b.status == 0
    _check_dispatch(bufs, xs, idxs, results, use_fp8, compact)

    # Experts: y = dequant(x) * (1 + global expert id); combine and compare.
    outs = []
    for d, b in enumerate(bufs):
        recv_x, scales, handle = results[d]
        with torch.cuda.device(b.device):
            if zero_copy:  # the "expert" writes straight into the region peers will read
                y = b.get_next_combine_buffer(handle).view(-1, hidden)
                y.zero_()
            else:
                y = torch.zeros(recv_x.shape[0], hidden, dtype=torch.bfloat16, device=b.device)
            offs, cnts = handle.expert_offsets.cpu(), handle.recv_count.cpu()
            for le in range(b.local_experts):
                s, c = int(offs[le]), int(cnts[le])
                if c == 0:
                    continue
                rows = dequant_fp8(recv_x[s : s + c], scales[s : s + c]) if use_fp8 else recv_x[s : s + c].float()
                y[s : s + c] = (rows * (1 + d * b.local_experts + le) * 0.01).to(torch.bfloat16)
            if compact:
                outs.append(b.combine(y, idxs[d], ws[d], handle))
            else:
                El, rows = b.local_experts, b.num_ranks * b.max_tokens
                outs.append(b.low_latency_combine(y.view(El, rows, hidden), idxs[d], ws[d], handle, zero_copy=zero_copy)[0])
    for b in bufs:
        torch.cuda.synchronize(b.device)
        assert b.status == 0
    for r, b in enumerate(bufs):
        x = xs[r]
        base = dequant_fp8(*per_token_cast_to_fp8(x)) if use_fp8 else x.float()
        want = torch.zeros(tokens, hidden, device=b.device)
        for k in range(topk):
            e = idxs[r][:, k]
            valid = (e >= 0).float().unsqueeze(1)
            yk = (base * ((1 + e.clamp(min=0)).float() * 0.01).unsqueeze(1)).to(torch.bfloat16).float()
            want += valid * ws[r][:, k].unsqueeze(1) * yk
        got, ref = outs[r].float(), want.to(torch.bfloat16).float()
        if not use_fp8:
            torch.testing.assert_close(got, ref, rtol=2e-2, atol=2e-2)
            continue
        # fp8: the kernel and PyTorch round x * (448 / amax) differently on exact ties, so a rare e4m3 code sits one
        # step apart (up to 1/8 of the value, and the same x feeds every term of a token): nearly all elements to
        # bf16 accuracy, every element to one fp8 step.
        err = (got - ref).abs()
        assert float((err <= 2e-2 + 2e-2 * ref.abs()).float().mean()) >= 0.999
        assert bool((err <= 2e-2 + 0.13 * ref.abs()).all())


@pytest.mark.parametrize("use_fp8", [True, False])
def test_rank_reduced_combine_single_rank(use_fp8):
    """Dispatch is given the weights, so the expert rank adds a token's rows up before one row returns."""
    bufs = _make_ranks(1, 8, 1024, 48, 4, tag=f"ep1rr_{int(use_fp8)}")
    for _ in range(3):  # both parity halves, and a slot reused with a new step tag
        _run(bufs, 48, 1024, 8, 4, use_fp8, True, rank_reduce=True)
    _run(bufs, 48, 1024, 8, 4, use_fp8, True)  # and back to the per-copy combine on the same buffer
    for b in bufs:
        b.destroy()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs (ranks wait on each other)")
@pytest.mark.parametrize("ranks", [2, 4])
def test_rank_reduced_combine_between_gpus(ranks):
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    bufs = _make_ranks(ranks, 8 * ranks, 1024, 64, 8, tag=f"eprr{ranks}")
    for _ in range(3):
        _run(bufs, 64, 1024, 8 * ranks, 8, True, True, rank_reduce=True)
    for b in bufs:
        b.destroy()


@pytest.mark.parametrize("use_fp8", [True, False])
@pytest.mark.parametrize("compact", [False, True])
def test_single_rank(use_fp8, compact):
    bufs = _make_ranks(1, 8, 1024, 48, 4, tag=f"ep1_{int(use_fp8)}{int(compact)}")
    _run(bufs, 48, 1024, 8, 4, use_fp8, compact)
    _run(bufs, 48, 1024, 8, 4, use_fp8, compact)  # second call: other parity half, counters were reset
    for b in bufs:
        b.destroy()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs (ranks wait on each other)")
@pytest.mark.parametrize("use_fp8", [True, False])
@pytest.mark.parametrize("compact", [False, True])
def test_multi_rank(use_fp8, compact):
    n = min(torch.cuda.device_count(), 8)
    bufs = _make_ranks(n, 8 * n, 2048, 64, 4, tag=f"epn_{int(use_fp8)}{int(compact)}")
    for _ in range(3):
        _run(bufs, 64, 2048, 8 * n, 4, use_fp8, compact)
    for b in bufs:
        b.barrier()
    for b in bufs:
        torch.cuda.synchronize(b.device)
        assert b.status == 0
        b.destroy()


@pytest.mark.parametrize("compact,pull,zero_copy", [(True, False, False), (True, True, True), (False, True, False), (False, None, True)])
def test_combine_push_pull_and_zero_copy(compact, pull, zero_copy):
    """Both combine algorithms on both layouts, with and without the caller writing into the exposed buffer."""
    n = min(torch.cuda.device_count(), 8)
    bufs = _make_ranks(n, 8 * n, 1024, 40, 4, tag=f"epc_{int(compact)}{pull}{int(zero_copy)}", combine_pull=pull)
    for _ in range(3):
        _run(bufs, 40, 1024, 8 * n, 4, True, compact, zero_copy=zero_copy)
    for b in bufs:
        torch.cuda.synchronize(b.device)
        assert b.status == 0
        b.destroy()


@pytest.mark.parametrize("compact", [False, True])
def test_combine_logfmt_matches_its_reference_model(compact):
    """Rows sent in the logarithmic 10-bit format decode to what the PyTorch model of the format
    predicts, and stay within a percent of the uncompressed result."""
    from nixl_b200.ops.logfmt import logfmt10_roundtrip

    n = min(torch.cuda.device_count(), 8)
    tokens, hidden, experts, topk = 40, 1024, 8 * n, 4
    bufs = _make_ranks(n, experts, hidden, tokens, topk, tag=f"eplog_{int(compact)}")
    for it in range(2):
        xs, idxs, ws = _inputs(bufs, tokens, hidden, experts, topk, seed=10 * it)
        for x in xs:
            x[1, :128] = 0          # a group of exact zeros
            x[2, 128:256] = 0.5     # a group with a single magnitude
            x[3, 300] = 0           # a zero inside a live group
        results = []
        for b, x, idx in zip(bufs, xs, idxs):
            with torch.cuda.device(b.device):
                if compact:
                    rx, _, handle = b.dispatch(x, idx, use_fp8=False)
                else:
                    recv, _, handle, _, _ = b.low_latency_dispatch(x, idx, use_fp8=False)
                    rx = recv.view(-1, hidden)
                results.append((rx, handle))
        outs = []
        for d, b in enumerate(bufs):
            rx, handle = results[d]
            with torch.cuda.device(b.device):
                y = (rx.float() * 0.37).to(torch.bfloat16)
                if compact:
                    outs.append(b.combine(y, idxs[d], ws[d], handle, use_logfmt=True))
                else:
                    outs.append(b.low_latency_combine(y.view(b.local_experts, -1, hidden), idxs[d], ws[d], handle, use_logfmt=True)[0])
        for b in bufs:
            torch.cuda.synchronize(b.device)
            assert b.status == 0
        for r, b in enumerate(bufs):
            yk = (xs[r].float() * 0.37).to(torch.bfloat16)
            model = torch.zeros(tokens, hidden, device=b.device)
            exact = torch.zeros(tokens, hidden, device=b.device)
            seen = logfmt10_roundtrip(yk)
            for k in range(topk):
                wk = (ws[r][:, k] * (idxs[r][:, k] >= 0).float()).unsqueeze(1)
                model += wk * seen
                exact += wk * yk.float()
            got = outs[r].float()
            # The model states the kernel's arithmetic bit for bit; what is left is the order of the fp32 sums.
            assert ((got - model).norm() / model.norm()).item() < 3e-3
            assert ((got - exact).norm() / exact.norm()).item() < 1e-2
            torch.testing.assert_close(got, model.to(torch.bfloat16).float(), rtol=1.6e-2, atol=1e-4)
            assert torch.all(got[1, :128] == 0)
            keep = (ws[r][2] * (idxs[r][2] >= 0).float()).sum().item()
            torch.testing.assert_close(got[2, 128:256], torch.full((128,), 0.5 * 0.37 * keep, device=b.device).to(torch.bfloat16).float(),
                                       rtol=1e-2, atol=1e-4)
    with pytest.raises(ValueError):
        bufs[0].low_latency_combine(torch.zeros(1), idxs[0], ws[0], results[0][1], use_logfmt=True, zero_copy=True)
    for b in bufs:
        b.destroy()


def test_throughput_only_buffer_is_smaller_and_rejects_low_latency_calls():
    dev = torch.device("cuda", 0)
    small = Buffer(0, 1, 8, 1024, 64, 2, device=dev, low_latency_mode=False)
    big = Buffer(0, 1, 8, 1024, 64, 2, device=dev, agent=small.agent)
    assert small.buffer.numel() < big.buffer.numel()
    x = torch.randn(64, 1024, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, 8, (64, 2), device=dev)
    with pytest.raises(ValueError):
        small.low_latency_dispatch(x, idx)
    rx, sc, h = small.dispatch(x, idx)
    torch.cuda.synchronize()
    assert int(h.recv_count.sum()) == 128 and small.status == 0


def test_ue8m0_scales_are_the_exponents_of_rounded_scales():
    dev = torch.device("cuda", 0)
    T, H, E, K = 40, 1024, 8, 2
    buf = Buffer(0, 1, E, H, T, K, device=dev)
    g = torch.Generator(device=dev).manual_seed(5)
    x = (torch.randn(T, H, device=dev, generator=g) * 3).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:K] for _ in range(T)]).long()
    (rx, packed), cnt, handle, _, _ = buf.low_latency_dispatch(x, idx, use_fp8=True, use_ue8m0=True)
    torch.cuda.synchronize()
    assert buf.status == 0 and packed.dtype == torch.int32 and packed.shape[-1] == H // 512
    want_q, want_s = per_token_cast_to_fp8(x, round_scale=True)
    scales = dequant_ue8m0(packed)  # [El, rows, H/128]
    info = handle.src_info.view(E, -1, 2)
    for le in range(E):
        for i in range(int(cnt[le])):
            t = int(info[le, i, 1]) // K
            assert torch.equal(scales[le, i], want_s[t]), (le, i)
            got = rx[le, i].view(torch.uint8).int()
            ref = want_q[t].view(torch.uint8).int()
            assert (got - ref).abs().max() <= 1
    buf.destroy()


def test_dispatch_ue8m0_feeds_block_scaled_gemm():
    """Throughput dispatch with exponent-byte scales straight into the block-scaled grouped GEMM, result into the
    exposed combine buffer, pull combine: the whole expert layer without a staging copy."""
    from nixl_b200.ops import from_ue8m0, grouped_gemm_mxfp8, quantize_weights_ue8m0

    dev = torch.device("cuda", 0)
    T, H, E, K, N = 96, 1024, 4, 2, 1024  # N = H so the outputs can go back through combine
    buf = Buffer(0, 1, E, H, T, K, device=dev, low_latency_mode=False)
    g = torch.Generator(device=dev).manual_seed(9)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    wts, idx = torch.topk(torch.softmax(torch.randn(T, E, device=dev, generator=g), -1), K, -1)
    idx, wts = idx.long().contiguous(), wts.float().contiguous()
    w = torch.randn(E, N, H, device=dev, generator=g) * 0.05
    wq, swb = quantize_weights_ue8m0(w)
    rx, packed, handle = buf.dispatch(x, idx, use_fp8=True, use_ue8m0=True)
    y = buf.get_next_combine_buffer(handle)
    grouped_gemm_mxfp8(rx[: buf.compact_rows], packed[: buf.compact_rows].contiguous(), wq, swb, handle.expert_offsets, handle.recv_count, out=y)
    out = buf.combine(y, idx, wts, handle)
    torch.cuda.synchronize()
    assert buf.status == 0
    q, s = per_token_cast_to_fp8(x, round_scale=True)
    xd = dequant_fp8(q, s)
    wd = (wq.float().view(E, N // 128, 128, H // 128, 128) * from_ue8m0(swb)[:, :, None, :, None]).view(E, N, H)
    want = torch.zeros(T, N, device=dev)
    for k in range(K):
        yk = torch.einsum("th,tnh->tn", xd, wd[idx[:, k]]).to(torch.bfloat16).float()
        want += wts[:, k : k + 1] * yk
    torch.testing.assert_close(out.float(), want.to(torch.bfloat16).float(), rtol=3e-2, atol=3e-2)
    buf.destroy()


def test_resize_and_utility_entry_points():
    dev = torch.device("cuda", 0)
    buf = Buffer(0, 1, 8, 1024, 32, 2, device=dev)
    assert Buffer.get_low_latency_buffer_size_hint(32, 1024, 1, 8, 2) == Buffer.get_low_latency_rdma_size_hint(32, 1024, 1, 8, 2)
    buf.set_num_sms(16)
    assert buf.num_sms == 16 and buf.get_dispatch_config()["num_sms"] == 16
    assert buf.get_local_buffer_tensor(torch.int32).numel() * 4 == buf.buffer.numel()
    x = torch.randn(32, 1024, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, 8, (32, 2), device=dev)
    buf.dispatch(x, idx)
    ev = buf.capture()
    ev.current_stream_wait()
    torch.cuda.synchronize()
    assert buf.status == 0
    before = buf.buffer.numel()
    buf.update_memory_buffers(1, 16)  # twice the local experts: a larger buffer, same agent
    assert buf.local_experts == 16 and buf.num_experts == 16 and buf.buffer.numel() > before and buf.num_sms == 16
    idx = torch.randint(0, 16, (32, 2), device=dev)
    rx, sc, h = buf.dispatch(x, idx)
    torch.cuda.synchronize()
    assert buf.status == 0 and int(h.recv_count.sum()) == 64
    buf.destroy()


def test_dispatch_layout_counts_match_torch():
    dev = torch.device("cuda", 0)
    buf = Buffer(0, 4, 32, 1024, 300, 6, device=dev, low_latency_mode=False)  # statistics need no peers
    g = torch.Generator(device=dev).manual_seed(3)
    idx = torch.stack([torch.randperm(32, device=dev, generator=g)[:6] for _ in range(300)]).long()
    idx[::7, 2] = -1
    per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx)
    torch.cuda.synchronize()
    valid = idx >= 0
    want_expert = torch.bincount(idx[valid], minlength=32)
    ranks = torch.where(valid, idx // 8, torch.full_like(idx, -1))
    want_in = torch.stack([(ranks == r).any(dim=1) for r in range(4)], dim=1)
    assert torch.equal(per_expert.long(), want_expert)
    assert torch.equal(in_rank, want_in)
    assert torch.equal(per_rank.long(), want_in.sum(dim=0))


def test_silent_rank_is_masked_not_waited_for():
    """Rank 1 exists but never launches: rank 0's waits run out (200 ms), rank 1 is masked and
    the status word says so; the GPU is idle again afterwards."""
    bufs = _make_ranks(2, 8, 1024, 16, 2, timeout_ms=200, tag="epmask")
    b0 = bufs[0]
    x = torch.randn(16, 1024, device=b0.device, dtype=torch.bfloat16)
    idx = torch.randint(0, 8, (16, 2), device=b0.device, dtype=torch.int64)
    with torch.cuda.device(b0.device):
        recv, cnt, handle, _, _ = b0.low_latency_dispatch(x, idx, use_fp8=True)
    torch.cuda.synchronize(b0.device)
    assert b0.status & 1
    assert b0.query_mask_buffer().tolist() == [0, 1]
    # Only rank 0's own tokens to its own experts are counted.
    assert int(cnt.sum()) == int((idx < 4).sum())
    b0.clean_mask_buffer()
    assert b0.status == 0 and b0.query_mask_buffer().tolist() == [0, 0]
    for b in bufs:
        b.destroy()


def test_dispatch_overlapped_with_grouped_gemm_matches_sequential():
    """Dispatch on a side stream + GEMM consuming arrival flags gives the same product as
    dispatch, wait, GEMM (single rank; both layouts)."""
    from nixl_b200.ops import grouped_gemm_fp8, quantize_weights

    T, H, E, K, N = 96, 1024, 8, 4, 256
    bufs = _make_ranks(1, E, H, T, K, tag="epgemm")
    b = bufs[0]
    xs, idxs, _ = _inputs(bufs, T, H, E, K, seed=5)
    wq, sw = quantize_weights(torch.randn(E, N, H, device=b.device) * 0.05)
    for low_latency in (True, False):
        if low_latency:
            (rx, sc), cnt, h, _, _ = b.low_latency_dispatch(xs[0], idxs[0])
            rx, sc = rx.view(-1, H), sc.view(-1, H // 128)
        else:
            rx, sc, h = b.dispatch(xs[0], idxs[0])
        torch.cuda.synchronize()
        want = grouped_gemm_fp8(rx.contiguous(), sc.contiguous(), wq, sw, h.expert_offsets, h.recv_count).clone()
        offs, cnts = h.expert_offsets.cpu().tolist(), h.recv_count.cpu().tolist()
        got, h2, _, _ = b.dispatch_gemm(xs[0], idxs[0], wq, sw, low_latency=low_latency)
        torch.cuda.synchronize()
        assert b.status == 0 and int(b._gemm_status.item()) == 0
        assert h2.recv_count.cpu().tolist() == cnts
        # Row order inside an expert may differ between two dispatches (slots are handed out by
        # atomics), so compare per expert as sorted multisets of rows.
        for e in range(E):
            s, c = offs[e], cnts[e]
            if c == 0:
                continue
            a_rows = want[s : s + c].float()
            b_rows = got[s : s + c].float()
            ka = a_rows.sum(dim=1).sort().values
            kb = b_rows.sum(dim=1).sort().values
            torch.testing.assert_close(ka, kb, rtol=1e-2, atol=1e-2)
    b.destroy()


def _ll_step(bufs, live, xs, idxs, ws, hidden):
    """One low-latency dispatch + combine on the ranks in `live`; returns their outputs."""
    res = {}
    for r in live:
        b = bufs[r]
        with torch.cuda.device(b.device):
            recv, cnt, handle, _, _ = b.low_latency_dispatch(xs[r], idxs[r], use_fp8=False)
            res[r] = (recv, handle)
    outs = {}
    for r in live:
        b = bufs[r]
        recv, handle = res[r]
        with torch.cuda.device(b.device):
            y = (recv.float() * 0.5).to(torch.bfloat16)
            outs[r] = b.low_latency_combine(y, idxs[r], ws[r], handle)[0]
    for r in live:
        torch.cuda.synchronize(bufs[r].device)
    return outs


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs (ranks wait on each other)")
def test_rank_leaves_between_steps_and_rejoins():
    """Scale down and up again, the scenario of the reference's elastic test: a rank is disconnected
    between steps (on the host, nothing of it in flight), the others go on without its experts, then
    it reconnects, catches up with the step counter and takes part again."""
    n = min(torch.cuda.device_count(), 4)
    tokens, hidden, topk = 24, 1024, 4
    experts = 4 * n
    bufs = _make_ranks(n, experts, hidden, tokens, topk, tag="epel", timeout_ms=3000)
    xs, idxs, ws = _inputs(bufs, tokens, hidden, experts, topk, seed=77)
    el = experts // n
    gone = n - 1

    def expect(r, masked_ranks):
        want = torch.zeros(tokens, hidden, device=bufs[r].device)
        yk = (xs[r].float() * 0.5).to(torch.bfloat16).float()
        for k in range(topk):
            e = idxs[r][:, k]
            ok = e >= 0
            for m in masked_ranks:
                ok = ok & (torch.div(e.clamp(min=0), el, rounding_mode="floor") != m)
            want += (ws[r][:, k] * ok.float()).unsqueeze(1) * yk
        return want.to(torch.bfloat16).float()

    everyone = list(range(n))
    outs = _ll_step(bufs, everyone, xs, idxs, ws, hidden)
    for r in everyone:
        assert bufs[r].status == 0
        torch.testing.assert_close(outs[r].float(), expect(r, []), rtol=2e-2, atol=2e-2)

    # The last rank leaves: the others learn of it on the host before their next launch.
    live = everyone[:-1]
    for r in live:
        bufs[r].disconnect_ranks([gone])
    for _ in range(2):
        outs = _ll_step(bufs, live, xs, idxs, ws, hidden)
        for r in live:
            assert bufs[r].status == 0  # nobody waited for the absent rank
            assert int(bufs[r].query_mask_buffer()[gone]) == 1
            torch.testing.assert_close(outs[r].float(), expect(r, [gone]), rtol=2e-2, atol=2e-2)

    # It comes back: fresh metadata both ways; the returning rank adopts the others' step counter.
    md = [b.local_metadata() for b in bufs]
    assert bufs[gone].epoch < bufs[0].epoch
    for r in live:
        bufs[r].connect_ranks([gone], metadata=md)
    bufs[gone].connect_ranks(live, metadata=md)
    assert bufs[gone].epoch == bufs[0].epoch
    outs = _ll_step(bufs, everyone, xs, idxs, ws, hidden)
    for r in everyone:
        assert bufs[r].status == 0 and int(bufs[r].query_mask_buffer().sum()) == 0
        torch.testing.assert_close(outs[r].float(), expect(r, []), rtol=2e-2, atol=2e-2)
    for b in bufs:
        b.destroy()
