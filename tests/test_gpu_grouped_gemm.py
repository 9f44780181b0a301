"""tcgen05 grouped fp8 GEMM against an fp32 PyTorch reference of the same product."""
import pytest
import torch

from nixl_b200.ops import (
    from_ue8m0,
    grouped_gemm_fp8,
    grouped_gemm_mxfp8,
    quantize_weights,
    quantize_weights_ue8m0,
    reference_grouped_gemm,
    to_ue8m0,
)
from nixl_b200.parallel import per_token_cast_to_fp8

pytestmark = pytest.mark.gpu


def _case(G, N, K, counts, gap=0, seed=0):
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(seed)
    starts, run = [], 0
    for c in counts:
        starts.append(run)
        run += c + gap
    rows = max(run, 1)
    x = torch.randn(rows, K, device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
    a, sa = per_token_cast_to_fp8(x)
    w = torch.randn(G, N, K, device=dev, generator=g) * 0.05
    wq, sw = quantize_weights(w)
    rs = torch.tensor(starts, dtype=torch.int32, device=dev)
    rc = torch.tensor(counts, dtype=torch.int32, device=dev)
    return a.contiguous(), sa.contiguous(), wq, sw, rs, rc


@pytest.mark.parametrize(
    "G,N,K,counts,gap",
    [
        (1, 128, 128, [128], 0),
        (1, 128, 512, [128], 0),
        (2, 256, 512, [200, 57], 0),
        (4, 256, 1024, [0, 300, 1, 129], 7),
        (3, 384, 7168, [64, 130, 33], 0),
    ],
)
def test_matches_reference(G, N, K, counts, gap):
    _check(G, N, K, counts, gap, tile_mode=1)


@pytest.mark.parametrize(
    "G,N,K,counts,gap",
    [
        (1, 256, 256, [256], 0),
        (1, 256, 1024, [100], 0),
        (2, 512, 512, [300, 57], 0),
        (4, 256, 1024, [0, 600, 1, 129], 5),
        (3, 512, 7168, [64, 257, 512], 0),
    ],
)
def test_cta_pair_tiles_match_reference(G, N, K, counts, gap):
    """256 x 256 tiles on CTA pairs: ragged groups, empty groups, rows that end inside either CTA's half."""
    _check(G, N, K, counts, gap, tile_mode=2)


def _check(G, N, K, counts, gap, tile_mode):
    a, sa, wq, sw, rs, rc = _case(G, N, K, counts, gap)
    out = grouped_gemm_fp8(a, sa, wq, sw, rs, rc, tile_mode=tile_mode)
    torch.cuda.synchronize()
    assert int(out._nixl_status.item()) == 0
    want = reference_grouped_gemm(a, sa, wq, sw, rs, rc)
    for g, (s, c) in enumerate(zip(rs.tolist(), rc.tolist())):
        if c == 0:
            continue
        got = out[s : s + c].float()
        ref = want[s : s + c]
        err = (got - ref).abs().max().item()
        scale = ref.abs().max().item() + 1e-6
        assert err / scale < 2e-2, (g, err, scale)
        cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
        assert cos > 0.999, (g, cos)


@pytest.mark.parametrize(
    "G,N,K,counts,gap",
    [
        (1, 256, 512, [256], 0),
        (2, 512, 1536, [300, 57], 0),
        (4, 256, 1024, [0, 600, 1, 129], 3),
        (3, 512, 7168, [64, 257, 512], 0),
    ],
)
def test_block_scaled_tiles_match_reference(G, N, K, counts, gap):
    """Power-of-two scales applied by the tensor core (UE8M0 bytes through TMEM): scales that differ per row,
    per 128-channel step and per weight block must all land on the right products."""
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(11)
    starts, run = [], 0
    for c in counts:
        starts.append(run)
        run += c + gap
    rows = max(run, 1)
    spread = torch.exp2(torch.randint(-6, 6, (rows, K // 128), device=dev, generator=g).float()).repeat_interleave(128, dim=1)
    x = (torch.randn(rows, K, device=dev, generator=g) * spread).to(torch.bfloat16)
    a, sa = per_token_cast_to_fp8(x, round_scale=True)
    wspread = torch.exp2(torch.randint(-3, 3, (G, N // 128, 1, K // 128, 1), device=dev, generator=g).float())
    w = (torch.randn(G, N // 128, 128, K // 128, 128, device=dev, generator=g) * 0.05 * wspread).reshape(G, N, K)
    wq, sw_bytes = quantize_weights_ue8m0(w)
    rs = torch.tensor(starts, dtype=torch.int32, device=dev)
    rc = torch.tensor(counts, dtype=torch.int32, device=dev)
    sa_bytes = to_ue8m0(sa)
    assert len(torch.unique(sa_bytes)) > 3 and torch.equal(from_ue8m0(sa_bytes), sa)
    out = grouped_gemm_mxfp8(a.contiguous(), sa_bytes, wq, sw_bytes, rs, rc)
    torch.cuda.synchronize()
    assert int(out._nixl_status.item()) == 0
    want = reference_grouped_gemm(a, sa, wq, from_ue8m0(sw_bytes), rs, rc)
    for s0, c in zip(starts, counts):
        if c == 0:
            continue
        got, ref = out[s0 : s0 + c].float(), want[s0 : s0 + c]
        assert (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-6) < 2e-2
        assert torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item() > 0.999


def test_block_scaled_gemm_rejects_unsupported_shapes():
    dev = torch.device("cuda:0")
    a = torch.zeros(128, 640, device=dev).to(torch.float8_e4m3fn)
    w = torch.zeros(1, 256, 640, device=dev).to(torch.float8_e4m3fn)
    rs, rc = torch.zeros(1, dtype=torch.int32, device=dev), torch.full((1,), 128, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        grouped_gemm_mxfp8(a, torch.zeros(128, 5, dtype=torch.uint8, device=dev), w, torch.zeros(1, 2, 5, dtype=torch.uint8, device=dev), rs, rc)
    with pytest.raises(ValueError):
        to_ue8m0(torch.tensor([3.0], device=dev))
