"""Each CUDA kernel alone against a plain float32 statement of the same operation, at sizes
other than the engine's (widths that are no power of two, odd row counts, every head size)."""
import math
import random

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module", autouse=True)
def _lib():
    from openinfer_b200.kernels import lib
    lib.load()
    torch.manual_seed(0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [24, 100, 1000])
def test_embedding(dtype, hidden):
    from openinfer_b200.kernels import ops
    vocab, n = 77, 13
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    ids = torch.randint(0, vocab, (n,), device=DEV, dtype=torch.int32)
    out = torch.empty(n, hidden, device=DEV, dtype=dtype)
    ops.embedding(out, table, ids)
    assert torch.equal(out, table[ids.long()])  # a bit-exact copy
    if dtype == torch.bfloat16:  # a table stored in 32-bit feeding a bfloat16 model
        t32 = table.float() * 1.001
        ops.embedding(out, t32, ids)
        assert torch.equal(out, t32[ids.long()].to(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [20, 96, 1000, 5120, 13000])
def test_rmsnorm_plain_add_and_gather(dtype, hidden):
    from openinfer_b200.kernels import ops
    rows, eps = 7, 3e-5
    x = (torch.randn(rows, hidden, device=DEV) * 3).to(dtype)
    w32 = 1 + 0.1 * torch.randn(hidden, device=DEV)
    for w in ([w32.to(dtype), w32] if dtype == torch.bfloat16 else [w32]):  # weight may be stored in 32-bit
        ref = plain.rms_norm(x.float().cpu(), w.float().cpu(), eps)
        out = torch.empty_like(x)
        ops.rmsnorm(out, x.clone(), w, eps)
        assert torch.allclose(out.float().cpu(), ref, **tol(dtype))
    w = w32.to(dtype)
    # weight offset: scale is (1 + w)
    out = torch.empty_like(x)
    ops.rmsnorm(out, x.clone(), w, eps, weight_offset=1.0)
    assert torch.allclose(out.float().cpu(), plain.rms_norm(x.float().cpu(), 1.0 + w.float().cpu(), eps), **tol(dtype))
    # fused residual add: x <- x + delta (stored), norm of the rounded sum
    delta = torch.randn(rows, hidden, device=DEV).to(dtype)
    xs = x.clone()
    ops.rmsnorm(out, xs, w, eps, delta=delta)
    summed = (x.float() + delta.float()).to(dtype)
    assert torch.equal(xs, summed)
    assert torch.allclose(out.float().cpu(), plain.rms_norm(summed.float().cpu(), w.float().cpu(), eps), **tol(dtype))
    # gathered rows (with repeats), with and without a pending delta; x is left alone
    idx = torch.tensor([6, 0, 0, 3], device=DEV, dtype=torch.int32)
    g = torch.empty(4, hidden, device=DEV, dtype=dtype)
    xs = x.clone()
    ops.rmsnorm(g, xs, w, eps, row_idx=idx)
    assert torch.allclose(g.float().cpu(), plain.rms_norm(x.float().cpu()[idx.long().cpu()], w.float().cpu(), eps), **tol(dtype))
    ops.rmsnorm(g, xs, w, eps, delta=delta, row_idx=idx)
    assert torch.equal(xs, x)
    assert torch.allclose(g.float().cpu(), plain.rms_norm(summed.float().cpu()[idx.long().cpu()], w.float().cpu(), eps), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [24, 100, 1111])
def test_silu_mul(dtype, inter):
    from openinfer_b200.kernels import ops
    rows = 5
    gu = (torch.randn(rows, 2 * inter, device=DEV) * 2).to(dtype)
    out = torch.empty(rows, inter, device=DEV, dtype=dtype)
    ops.silu_mul(out, gu)
    g, u = gu.float()[:, :inter], gu.float()[:, inter:]
    assert torch.allclose(out.float(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 100, 33), (65, 129, 17), (130, 64, 300)])
def test_gemm_generic(dtype, M, N, K):
    from openinfer_b200.kernels import ops
    a = torch.randn(M, K, device=DEV).to(dtype)
    w = torch.randn(N, K, device=DEV).to(dtype)
    out = torch.empty(M, N, device=DEV, dtype=dtype)
    ops.gemm_generic(out, a, w)
    ref = a.double() @ w.double().t()
    assert torch.allclose(out.double(), ref, atol=1e-4 if dtype == torch.float32 else 0.15, rtol=1e-5 if dtype == torch.float32 else 2e-2)
    # float32 output from bfloat16 operands, strided input rows, mixed operand types
    big = torch.randn(M, K + 8, device=DEV).to(dtype)
    o32 = torch.empty(M, N, device=DEV, dtype=torch.float32)
    ops.gemm_generic(o32, big[:, :K], w.float())
    assert torch.allclose(o32.double(), big[:, :K].double() @ w.float().double().t(), atol=1e-4, rtol=1e-5)
    # a row's result does not depend on the other rows (batch invariance, bit for bit)
    one = torch.empty(1, N, device=DEV, dtype=dtype)
    ops.gemm_generic(one, a[M - 1:], w)
    assert torch.equal(one[0], out[M - 1])


def _rope_ref(x, positions, rot, theta, w, eps, offset):
    """plain: per-head norm then rotate-half over the first `rot` dims; x [T, heads, hd] float32 cpu"""
    if w is not None:
        x = plain.rms_norm(x, offset + w, eps)
    if rot:
        cos, sin = plain.rope_tables(rot, theta, positions)
        x = torch.cat([plain.apply_rope(x[..., :rot], cos, sin), x[..., rot:]], dim=-1)
    return x


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,rot,norm", [(4, 2, 16, 16, True), (6, 2, 32, 32, True), (5, 1, 64, 32, True),
                                                (3, 3, 128, 128, False), (2, 1, 256, 0, True), (7, 7, 48, 48, True)])
def test_qk_norm_rope_kv_write(dtype, nq, nkv, hd, rot, norm):
    from openinfer_b200.kernels import ops
    from openinfer_b200.parts.position import RotaryEncoding
    from openinfer_b200.parts.spec import PositionSpec
    T, P, pages, theta, eps, max_pos = 11, 4, 9, 5000.0, 1e-5, 64
    width = (nq + 2 * nkv) * hd
    qkv = torch.randn(T, width + 8, device=DEV).to(dtype)[:, :width]  # a row stride wider than the row
    src = qkv.clone().float().cpu()
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 40, 41, 63, 17], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 7, 12, 13, 14, 0, 1, 35, -1], dtype=torch.int32)  # -1: a padding row
    qw = (1 + 0.1 * torch.randn(hd)).to(dtype) if norm else None
    kw = (1 + 0.1 * torch.randn(hd)).to(dtype) if norm else None
    cos = sin = None
    if rot:
        cos, sin = RotaryEncoding(PositionSpec("rope", rot, theta, max_pos)).rotation_tables(torch.device(DEV))
    cache = torch.zeros(pages, 2, 2, P, nkv, hd, device=DEV, dtype=dtype)  # [pages, layers, k/v, P, nkv, hd]
    layer = 1
    ops.qk_norm_rope_kv(qkv, nq, nkv, hd, q_norm_w=qw.to(DEV) if norm else None, k_norm_w=kw.to(DEV) if norm else None,
                        eps=eps, weight_offset=0.0, cos=cos, sin=sin, positions=positions.to(DEV), slots=slots.to(DEV),
                        k_cache=cache[:, layer, 0], v_cache=cache[:, layer, 1], page_stride=cache.stride(0), page_size=P)
    q_ref = _rope_ref(src[:, : nq * hd].view(T, nq, hd), positions, rot, theta, qw.float() if norm else None, eps, 0.0)
    k_ref = _rope_ref(src[:, nq * hd: (nq + nkv) * hd].view(T, nkv, hd), positions, rot, theta, kw.float() if norm else None, eps, 0.0)
    v_ref = src[:, (nq + nkv) * hd:].view(T, nkv, hd)
    t = tol(dtype)
    assert torch.allclose(qkv[:, : nq * hd].float().cpu().view(T, nq, hd), q_ref, **t)
    assert torch.equal(qkv[:, nq * hd:].float().cpu(), src[:, nq * hd:])  # k, v inputs are not touched
    flat = cache[:, layer].float().cpu()  # [pages, 2, P, nkv, hd]
    for i in range(T):
        s = int(slots[i])
        if s < 0:
            continue
        assert torch.allclose(flat[s // P, 0, s % P], k_ref[i], **t), f"k row {i}"
        assert torch.allclose(flat[s // P, 1, s % P], v_ref[i].to(dtype).float(), atol=0, rtol=0), f"v row {i}"
    written = {int(s) for s in slots if s >= 0}
    for s in range(pages * P):
        if s not in written:
            assert flat[s // P, :, s % P].abs().sum() == 0, f"slot {s} was written"
    assert cache[:, 0].abs().sum() == 0  # the other layer of the page is untouched


def _paged(k, v, P, order, dtype, pages_total):
    """Put [S, nkv, hd] keys/values into pages in the given page order. Returns cache, block table row."""
    S, nkv, hd = k.shape
    cache = torch.zeros(pages_total, 1, 2, P, nkv, hd, dtype=dtype)
    for j in range(S):
        cache[order[j // P], 0, 0, j % P] = k[j].to(dtype)
        cache[order[j // P], 0, 1, j % P] = v[j].to(dtype)
    return cache


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,P,window", [
    (4, 2, 16, 8, None), (6, 2, 32, 16, None), (3, 1, 64, 4, 7), (8, 8, 128, 16, None), (5, 5, 256, 2, 33),
    (12, 4, 48, 16, None), (32, 8, 128, 16, 100), (2, 1, 8, 1, None)])
def test_attention_generic(dtype, nq, nkv, hd, P, window):
    """Two requests in one batch: a prompt portion over a cached prefix, and a single decoded token."""
    from openinfer_b200.kernels import ops
    torch.manual_seed(nq * 100 + hd)
    S0, new0, S1 = 70, 9, 131          # request 0: 61 cached + 9 new rows; request 1: 130 cached + 1 new
    scale = 1.0 / math.sqrt(hd)
    pages_total = 80
    perm = torch.randperm(pages_total).tolist()
    n0, n1 = -(-S0 // P), -(-S1 // P)
    if n0 + n1 > pages_total:
        pages_total = n0 + n1 + 3
        perm = torch.randperm(pages_total).tolist()
    order0, order1 = perm[:n0], perm[n0: n0 + n1]
    ks = [torch.randn(S, nkv, hd) for S in (S0, S1)]
    vs = [torch.randn(S, nkv, hd) for S in (S0, S1)]
    qs = [torch.randn(S, nq, hd) for S in (S0, S1)]
    cache = _paged(ks[0], vs[0], P, order0, dtype, pages_total)
    c1 = _paged(ks[1], vs[1], P, order1, dtype, pages_total)
    cache = (cache + c1).to(DEV)
    bt = torch.zeros(2, max(n0, n1), dtype=torch.int32)
    bt[0, :n0] = torch.tensor(order0)
    bt[1, :n1] = torch.tensor(order1)
    rows = [(0, p) for p in range(S0 - new0, S0)] + [(1, S1 - 1)]
    q = torch.stack([qs[r][p] for r, p in rows]).to(dtype)              # [T, nq, hd]
    wide = torch.zeros(len(rows), nq * hd + 2 * nkv * hd, dtype=dtype)  # q lives in a wider buffer
    wide[:, : nq * hd] = q.view(len(rows), -1)
    wide = wide.to(DEV)
    out = torch.empty(len(rows), nq * hd, device=DEV, dtype=dtype)
    ops.attention_generic(wide[:, : nq * hd], out, cache[:, 0, 0], cache[:, 0, 1], cache.stride(0), P, bt.to(DEV),
                          torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV),
                          torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV), nq, nkv, hd, scale, window)
    for i, (r, p) in enumerate(rows):
        kk, vv = ks[r].to(dtype).float(), vs[r].to(dtype).float()
        qq = torch.zeros(p + 1, nq, hd)
        qq[p] = q[i].float()
        ref = plain.causal_attention(qq, kk[: p + 1], vv[: p + 1], scale, window)[p]
        assert torch.allclose(out[i].float().cpu().view(nq, hd), ref, **tol(dtype)), f"row {i} (request {r}, position {p})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """One key among hundreds is made to stand out (scaled query and key): the output must be
    that key's value, wherever in the cache it lies: first position, a page's edge, mid-page."""
    from openinfer_b200.kernels import ops
    nq, nkv, hd, P, S = 2, 1, 32, 16, 600
    for far in (0, 15, 16, 17, 255, 256, 300, 598, 599):
        k = torch.randn(S, nkv, hd) * 0.1
        v = torch.randn(S, nkv, hd)
        q = torch.randn(1, nq, hd) * 0.1
        direction = torch.randn(hd)
        direction /= direction.norm()
        k[far, 0] = direction * 12.0
        q[0, :] = direction * 12.0 * math.sqrt(hd) / 2       # score = 72 * ... far above the rest
        order = torch.randperm(40).tolist()
        cache = _paged(k, v, P, order, dtype, 40).to(DEV)
        bt = torch.tensor([order[: -(-S // P)]], dtype=torch.int32, device=DEV)
        out = torch.empty(1, nq * hd, device=DEV, dtype=dtype)
        ops.attention_generic(q.view(1, -1).to(dtype).to(DEV), out, cache[:, 0, 0], cache[:, 0, 1], cache.stride(0), P, bt,
                              torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([S - 1], dtype=torch.int32, device=DEV),
                              nq, nkv, hd, 1.0 / math.sqrt(hd), None)
        want = v[far, 0].to(dtype).float()
        for h in range(nq):
            assert torch.allclose(out[0].float().cpu().view(nq, hd)[h], want, atol=2e-2), f"far key at {far}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(dtype):
    """The key just outside the window is made huge: it must not be seen; the one just inside must."""
    from openinfer_b200.kernels import ops
    nq, nkv, hd, P, S, W = 1, 1, 16, 4, 50, 9
    for inside in (False, True):
        k = torch.randn(S, nkv, hd) * 0.1
        v = torch.randn(S, nkv, hd)
        d = torch.zeros(hd)
        d[0] = 1.0
        pos = S - 1
        edge = pos - W + (1 if inside else 0)   # pos - W + 1 is the oldest visible key
        k[edge, 0] = d * 20
        q = (d * 20).view(1, 1, hd)
        order = list(range(13))
        cache = _paged(k, v, P, order, dtype, 13).to(DEV)
        bt = torch.tensor([order], dtype=torch.int32, device=DEV)
        out = torch.empty(1, hd, device=DEV, dtype=dtype)
        ops.attention_generic(q.view(1, -1).to(dtype).to(DEV), out, cache[:, 0, 0], cache[:, 0, 1], cache.stride(0), P, bt,
                              torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([pos], dtype=torch.int32, device=DEV),
                              nq, nkv, hd, 1.0, W)
        close = torch.allclose(out[0].float().cpu(), v[edge, 0].to(dtype).float(), atol=2e-2)
        assert close == inside


def test_argmax_ties_and_odd_vocab():
    from openinfer_b200.kernels import ops
    for vocab in (5, 1000, 151936 // 7):
        logits = torch.randn(6, vocab, device=DEV)
        logits[1, vocab // 2] = 50.0
        logits[2, :] = 1.0                       # all tied: lowest index
        logits[3, [vocab - 1, 2]] = 60.0         # tie between two: lowest index
        logits[4, vocab - 1] = 70.0
        out = torch.empty(6, dtype=torch.int32, device=DEV)
        ops.argmax(out, logits)
        ref = [int(torch.argmax(logits[0])), vocab // 2, 0, 2, vocab - 1, int(torch.argmax(logits[5]))]
        assert out.tolist() == ref
        wide = torch.randn(3, vocab + 5, device=DEV)[:, :vocab]  # strided rows
        out3 = torch.empty(3, dtype=torch.int32, device=DEV)
        ops.argmax(out3, wide)
        assert out3.tolist() == torch.argmax(wide, dim=-1).tolist()


@pytest.fixture(params=[True, False], ids=["clusters", "one-block"])
def sample_clusters(request):
    """Both ways through the sampler: a cluster of CTAs per row where the row allows it, and one block per row."""
    from openinfer_b200.kernels import ops
    ops.sample_use_clusters(request.param)
    yield request.param
    ops.sample_use_clusters(True)


@pytest.mark.parametrize("vocab", [50, 52, 384, 5000, 30001, 30004])
def test_sample_matches_plain_distribution(vocab, sample_clusters):
    """The kept set and the drawn token follow the plain statement of temperature / top-k /
    top-p / min-p, for uniform numbers across [0, 1). Vocabularies that are multiples of 4 go to the
    clusters (30004: the flat rows are then left to the one-block kernel), the others to one block."""
    from openinfer_b200.kernels import ops
    torch.manual_seed(vocab)
    settings = [(0.8, -1, 1.0, 0.0), (1.0, 5, 1.0, 0.0), (0.7, -1, 0.9, 0.0), (1.3, 20, 0.8, 0.0),
                (1.0, -1, 1.0, 0.1), (0.9, 10, 0.95, 0.05), (1.0, -1, 0.01, 0.0)]
    us = [0.0, 0.001, 0.25, 0.5, 0.75, 0.999, 0.9999999]
    logits = torch.randn(len(settings), vocab) * 2.0
    if vocab > 5000:
        # more values than the kernel's shared-memory list of candidates holds: peaked rows find their thresholds
        # in the list, the flat ones (spread 0.05) must fall back to scanning the vocabulary; rows 1 and 5 get
        # many exact ties at the top
        logits[2] *= 0.025
        logits[3] *= 0.025
        logits[1, :6000] = 9.0
        logits[5, ::3] = 7.0
    for u in us:
        rows = len(settings)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        scratch = torch.empty(rows * vocab, device=DEV)
        ops.sample(out, logits.to(DEV), scratch,
                   torch.tensor([s[0] for s in settings], device=DEV), torch.tensor([max(s[1], 0) for s in settings], dtype=torch.int32, device=DEV),
                   torch.tensor([s[2] for s in settings], device=DEV), torch.tensor([s[3] for s in settings], device=DEV),
                   torch.full((rows,), u, device=DEV))
        for r, (t, k, p, mp) in enumerate(settings):
            dist = plain.sampling_distribution(logits[r], t, k, p, mp)
            tok = int(out[r])
            assert dist[tok] > 0, f"setting {settings[r]} u={u}: token {tok} is outside the kept set"
            cdf = torch.cumsum(dist, 0)
            lo = float(cdf[tok] - dist[tok])
            assert lo - 1e-4 <= u <= float(cdf[tok]) + 1e-4, f"setting {settings[r]} u={u}: token {tok} covers [{lo}, {float(cdf[tok])}]"


def test_sample_when_the_estimate_of_the_candidate_list_is_wrong(sample_clusters):
    """The kernel places the cut of its shared-memory list from a histogram of one value in eight (the first of
    every other group of four per thread). 5,000 equal large values at places that are never counted make that
    estimate miss them all: the list overflows, is dropped, and the thresholds come from the whole row."""
    from openinfer_b200.kernels import ops
    torch.manual_seed(5)
    vocab = 151936
    settings = [(1.0, 10, 1.0, 0.0), (1.0, -1, 0.5, 0.0), (0.8, 7000, 0.9, 0.0)]
    logits = torch.randn(len(settings), vocab) * 0.01
    hot = torch.arange(vocab)[torch.arange(vocab) % 4 == 1][:5000]
    logits[:, hot] = 5.0
    logits[2, hot[:100]] = 6.0
    rows = len(settings)
    for u in (0.0, 0.3, 0.77, 0.9999):
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        scratch = torch.empty(rows * vocab, device=DEV)
        ops.sample(out, logits.to(DEV), scratch,
                   torch.tensor([s[0] for s in settings], device=DEV), torch.tensor([max(s[1], 0) for s in settings], dtype=torch.int32, device=DEV),
                   torch.tensor([s[2] for s in settings], device=DEV), torch.tensor([s[3] for s in settings], device=DEV),
                   torch.full((rows,), u, device=DEV))
        for r, (t, k, p, mp) in enumerate(settings):
            dist = plain.sampling_distribution(logits[r], t, k, p, mp)
            tok = int(out[r])
            assert dist[tok] > 0, f"setting {settings[r]} u={u}: token {tok} is outside the kept set"
            cdf = torch.cumsum(dist.double(), 0)
            lo = float(cdf[tok] - dist[tok])
            assert lo - 1e-4 <= u <= float(cdf[tok]) + 1e-4, f"setting {settings[r]} u={u}: token {tok} covers [{lo}, {float(cdf[tok])}]"


# ---------------------------------------------------------------------------
# the tensor-core attention kernel (bfloat16; prompt tiles and split-KV decode)
# ---------------------------------------------------------------------------
class _FakeCache:
    def __init__(self, page_size):
        self.page_size = page_size


class _FakeCtx:
    """What the attention dispatcher reads of a StepContext."""

    def __init__(self, q_lens, kv_lens, P):
        self.q_lens_host, self.kv_lens_host = list(q_lens), list(kv_lens)
        self.num_tokens = sum(q_lens)
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + n)
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=DEV)
        self.token_req = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
        self.positions = torch.tensor([kv - n + i for n, kv in zip(q_lens, kv_lens) for i in range(n)], dtype=torch.int32, device=DEV)
        self.cache = _FakeCache(P)
        self.scratch = {}


class _FakeGroup:
    def __init__(self, block_table, kv_lens):
        self.block_table = block_table
        self.kv_lens = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)


def _pages_in_runs(total_pages, seed):
    """All page ids, in runs of 1 to 9 consecutive ids that come in random order: some groups of neighbouring
    table entries are consecutive pages, some are not, some runs end in the middle of a tile."""
    rng = random.Random(seed)
    runs, at = [], 0
    while at < total_pages:
        n = min(total_pages - at, rng.randint(1, 9))
        runs.append(list(range(at, at + n)))
        at += n
    rng.shuffle(runs)
    return [p for run in runs for p in run]


def _mma_case(nq, nkv, hd, P, window, q_lens, kv_lens, seed=0, force_splits=None, page_runs=False):
    from openinfer_b200.kernels import attention as A
    torch.manual_seed(seed)
    dtype = torch.bfloat16
    n_req = len(q_lens)
    pages_needed = [-(-kv // P) for kv in kv_lens]
    total_pages = sum(pages_needed) + 5
    perm = _pages_in_runs(total_pages, seed) if page_runs else torch.randperm(total_pages).tolist()
    cache = torch.zeros(total_pages, 2, 2, P, nkv, hd, dtype=dtype)   # two layers per page; layer 1 is used
    bt = torch.zeros(n_req, max(pages_needed), dtype=torch.int32)
    ks, vs, at = [], [], 0
    for b, kv in enumerate(kv_lens):
        order = perm[at: at + pages_needed[b]]
        at += pages_needed[b]
        bt[b, : len(order)] = torch.tensor(order)
        k, v = torch.randn(kv, nkv, hd).to(dtype), torch.randn(kv, nkv, hd).to(dtype)
        for j in range(kv):
            cache[order[j // P], 1, 0, j % P] = k[j]
            cache[order[j // P], 1, 1, j % P] = v[j]
        ks.append(k.float())
        vs.append(v.float())
    cache = cache.to(DEV)
    T = sum(q_lens)
    q = torch.randn(T, nq, hd).to(dtype)
    wide = torch.zeros(T, (nq + 2 * nkv) * hd, dtype=dtype)
    wide[:, : nq * hd] = q.view(T, -1)
    wide = wide.to(DEV)
    ctx = _FakeCtx(q_lens, kv_lens, P)
    grp = _FakeGroup(bt.to(DEV), kv_lens)
    if force_splits:
        old = A.plan_items

        def forced(ql, kl, group, nkv_, window_, sm, decode_kernel=True, rows_per_cta=None, whole_tiles_kernel=False):
            if force_splits == "tiles":     # decode rows through the tile kernel, cut into slices
                return old(ql, kl, group, nkv_, window_, 10 ** 6, decode_kernel=False, rows_per_cta=rows_per_cta)
            if force_splits == "tiles_whole":
                return old(ql, kl, group, nkv_, window_, 1, decode_kernel=False, rows_per_cta=rows_per_cta)
            return old(ql, kl, group, nkv_, window_, 10 ** 6 if force_splits == "max" else 1, rows_per_cta=rows_per_cta)
        A.plan_items = forced
    try:
        out = torch.full((T, nq * hd), float("nan"), device=DEV, dtype=dtype)
        ran = A.attention_mma(wide[:, : nq * hd], out, cache[:, 1, 0], cache[:, 1, 1], cache.stride(0), ctx, grp,
                              nq, nkv, hd, 1.0 / math.sqrt(hd), window)
    finally:
        if force_splits:
            A.plan_items = old
    assert ran
    assert A.tcgen05_status() == 0, "a bounded wait ran out in the tcgen05 attention kernel"
    plan = next(iter(ctx.scratch.values()))
    step = [v for k, v in ctx.scratch.items() if k[0] == "attention_step"][0]
    if (A.USE_TCGEN05 and hd == 128 and plan.rows_per_cta == 128 and 128 % (nq // nkv) == 0 and P >= 16 and P & (P - 1) == 0
            and plan.num_tile_items):
        assert step.use_tcgen05, "the tcgen05 kernel covers this shape and did not run"
    scale = 1.0 / math.sqrt(hd)
    row = 0
    for b, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        qq = torch.zeros(kv, nq, hd)
        qq[kv - n:] = q[row: row + n].float()
        ref = plain.causal_attention(qq, ks[b], vs[b], scale, window)[kv - n:]
        got = out[row: row + n].float().cpu().view(n, nq, hd)
        assert torch.isfinite(got).all(), f"request {b}: unwritten or non-finite output"
        err = (got - ref).abs()
        assert err.max() < 3e-2, f"request {b} (q {n}, kv {kv}): max err {err.max():.4f} at row {int(err.amax(dim=(1, 2)).argmax())}"
        row += n
    return plan


@pytest.mark.parametrize("tcgen05", [True, False])
@pytest.mark.parametrize("nq,nkv,hd,P,window", [
    (32, 8, 128, 16, None), (6, 2, 32, 16, None), (8, 2, 64, 8, None), (3, 1, 128, 4, None),
    (16, 16, 64, 16, None), (5, 1, 32, 1, None), (8, 2, 128, 16, 100), (4, 2, 64, 16, 17), (64, 1, 32, 16, None),
    (2, 2, 128, 32, None), (16, 2, 128, 64, 70), (4, 1, 128, 128, None)])
def test_attention_mma_mixed_batch(nq, nkv, hd, P, window, tcgen05, monkeypatch):
    """Prompt portions over cached prefixes beside single decoded tokens, in one launch; the tiles
    through the tcgen05 kernel where it covers the shape, and through the mma.sync kernel."""
    from openinfer_b200.kernels import attention as A
    monkeypatch.setattr(A, "USE_TCGEN05", tcgen05)
    q_lens = [9, 1, 70, 1, 33, 2]
    kv_lens = [70, 131, 70, 1, 300, 65]
    plan = _mma_case(nq, nkv, hd, P, window, q_lens, kv_lens)
    assert plan.rows_per_cta == (128 if 70 * (nq // nkv) >= 128 else 64)
    # short portions only: the small tile
    plan = _mma_case(nq, nkv, hd, P, window, [3, 1, 2], [70, 131, 300])
    assert plan.rows_per_cta == (64 if 3 * (nq // nkv) < 128 else 128)


@pytest.mark.parametrize("nq,nkv,hd", [(32, 8, 128), (6, 2, 32), (8, 1, 64)])
@pytest.mark.parametrize("window", [None, 200])
def test_attention_mma_split_kv_decode(nq, nkv, hd, window, monkeypatch):
    """Decode rows whose keys are cut into slices and merged; contexts around tile edges."""
    from openinfer_b200.kernels import attention as A
    kv_lens = [1, 63, 64, 65, 127, 128, 129, 700, 1025]
    long = kv_lens + [2100]
    monkeypatch.setattr(A, "DECODE_MAX_SPLITS", 64)     # more slices than the planner uses: the second kernel merges
    plan = _mma_case(nq, nkv, hd, 16, window, [1] * len(long), long, force_splits="max")
    monkeypatch.setattr(A, "DECODE_MAX_SPLITS", 32)
    # the decode kernel, 64 slices: too many CTAs per row for a cluster, merged by the second kernel
    assert plan.num_decode_items and plan.max_splits == 64 and not plan.num_tile_items and not plan.decode_merge_in_kernel
    plan = _mma_case(nq, nkv, hd, 16, window, [1] * len(kv_lens), kv_lens)
    # as planned for this GPU: 16 or 32 slices, the 4 or 8 CTAs of a row merge through distributed shared memory
    assert plan.num_decode_items and plan.max_splits in (16, 32) and plan.decode_merge_in_kernel
    plan = _mma_case(nq, nkv, hd, 16, window, [1] * len(kv_lens), kv_lens, force_splits="none")
    assert plan.num_decode_items and plan.max_splits == 4 and plan.decode_merge_in_kernel   # four slices: one CTA per row
    plan = _mma_case(nq, nkv, hd, 16, window, [1] * len(kv_lens), kv_lens, force_splits="tiles")
    assert plan.tile_split and not plan.num_decode_items                                 # the tile kernel, sliced
    plan = _mma_case(nq, nkv, hd, 16, window, [1] * len(kv_lens), kv_lens, force_splits="tiles_whole")
    assert not plan.tile_split and plan.max_splits == 1


def test_attention_mma_split_prompt_portion():
    """A short portion over a long prefix is also cut into slices when the grid is small."""
    plan = _mma_case(8, 2, 64, 16, None, [5, 3], [900, 400], force_splits="max")
    assert plan.tile_split
    # beside decode rows the tiles stay whole (one merge pass, after the decode kernel)
    plan = _mma_case(8, 2, 64, 16, None, [5, 1], [900, 400], force_splits="max")
    assert not plan.tile_split and plan.num_decode_items


@pytest.mark.parametrize("nq,nkv,P,window", [(32, 8, 16, None), (8, 4, 64, None), (4, 2, 16, 200), (16, 1, 32, None)])
def test_attention_tcgen05_with_key_slices(nq, nkv, P, window):
    """Prompt tiles whose keys are cut into slices (a grid that would leave SMs idle) through the tcgen05 kernel:
    every slice leaves its normalised partial result and log-sum-exp in scratch, a second kernel merges them.
    Portions over long prefixes, slices that come out empty, a window."""
    from openinfer_b200.kernels import attention as A
    for q_lens, kv_lens in (([260, 70], [900, 330]), ([33], [1200]), ([150, 40, 129], [150, 1000, 640])):
        plan = _mma_case(nq, nkv, 128, P, window, q_lens, kv_lens, force_splits="max")
        assert plan.tile_split and plan.max_splits > 1     # _mma_case checks that the tcgen05 kernel ran where it covers the shape
        assert A.tcgen05_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("nq,nkv,P,window", [(8, 2, 16, None), (4, 4, 32, None), (16, 2, 16, 100), (8, 8, 64, None)])
def test_attention_tcgen05_with_runs_of_consecutive_pages(nq, nkv, P, window):
    """Pages whose ids follow one another are fetched with ONE box per 64-key tile, the others page by page; tables
    that mix both (runs of 1 to 9 pages in random order, so runs begin and end inside tiles), and the identity table
    of a fresh pool."""
    for seed, (q_lens, kv_lens) in enumerate((([300, 77], [300, 333]), ([129], [1100]), ([64, 200, 5], [640, 200, 390]))):
        _mma_case(nq, nkv, 128, P, window, q_lens, kv_lens, seed=seed, page_runs=True)
    from openinfer_b200.kernels import attention as A
    assert A.tcgen05_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("nq,nkv,hd", [(8, 2, 128), (4, 4, 64)])
def test_attention_decode_with_64_and_128_key_slices_at_long_contexts(nq, nkv, hd):
    """Decode rows over 13,000 and 25,000 keys: when 32 slices a row leave SMs idle such rows are cut into 64 or
    128 slices, whose partial results go through global memory and the merge kernel (128 is the most it takes).
    One far key is made to stand out (its k aligned with q), so a slice that is lost or merged with a wrong
    weight shows. Reference: the row's softmax over all keys in float64."""
    from openinfer_b200.kernels import attention as A
    P = 16
    for kv_lens, want_splits in (([13000], 64), ([13000, 12500], 64), ([25000, 13000], 128)):
        torch.manual_seed(len(kv_lens) + want_splits)
        pages_needed = [-(-kv // P) for kv in kv_lens]
        total_pages = sum(pages_needed) + 3
        perm = torch.randperm(total_pages)
        cache = torch.zeros(total_pages, 2, P, nkv, hd, dtype=torch.bfloat16)
        bt = torch.zeros(len(kv_lens), max(pages_needed), dtype=torch.int32)
        q = torch.randn(len(kv_lens), nq, hd).to(torch.bfloat16)
        ks, vs, at = [], [], 0
        for b, kv in enumerate(kv_lens):
            order = perm[at: at + pages_needed[b]]
            at += pages_needed[b]
            bt[b, : len(order)] = order.to(torch.int32)
            k, v = torch.randn(kv, nkv, hd).to(torch.bfloat16), torch.randn(kv, nkv, hd).to(torch.bfloat16)
            far = 37 + 1000 * b        # a key in an early slice that outweighs the others for head 0
            k[far, 0] = (q[b, 0].float() * 2.0).to(torch.bfloat16)
            pad = pages_needed[b] * P - kv
            kp = torch.cat([k, torch.zeros(pad, nkv, hd, dtype=torch.bfloat16)]).view(-1, P, nkv, hd)
            vp = torch.cat([v, torch.zeros(pad, nkv, hd, dtype=torch.bfloat16)]).view(-1, P, nkv, hd)
            cache[order, 0] = kp
            cache[order, 1] = vp
            ks.append(k.double())
            vs.append(v.double())
        cache = cache.to(DEV)
        ctx = _FakeCtx([1] * len(kv_lens), kv_lens, P)
        grp = _FakeGroup(bt.to(DEV), kv_lens)
        out = torch.full((len(kv_lens), nq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
        old = A._sm_count
        A._sm_count = lambda device: 10 ** 6      # as on a GPU that 32 slices a row never fill
        try:
            assert A.attention_mma(q.view(len(kv_lens), -1).to(DEV), out, cache[:, 0], cache[:, 1], cache.stride(0), ctx, grp,
                                   nq, nkv, hd, 1.0 / math.sqrt(hd), None)
        finally:
            A._sm_count = old
        plan = next(iter(ctx.scratch.values()))
        assert plan.max_splits == want_splits and not plan.decode_merge_in_kernel
        group = nq // nkv
        for b, kv in enumerate(kv_lens):
            for h in range(nq):
                s = (ks[b][:, h // group] @ q[b, h].double()) / math.sqrt(hd)
                ref = torch.softmax(s, dim=0) @ vs[b][:, h // group]
                got = out[b].float().cpu().view(nq, hd)[h].double()
                err = (got - ref).abs().max().item()
                assert err <= 2e-2 * max(1.0, ref.abs().max().item()), f"kv {kv} head {h}: {err}"
            # the far key carries most of head 0's weight: its value dominates the output
            far = 37 + 1000 * b
            assert (out[b].float().cpu().view(nq, hd)[0] - vs[b][far, 0].float()).abs().max().item() < 0.35


def test_attention_mma_plan():
    from openinfer_b200.kernels.attention import decode_splits, plan_items
    # decode rows: 32 slices at most (what a cluster merges), 64 and 128 for long rows that leave SMs idle otherwise,
    # never in a step that also brings prompt portions (the merge scratch is indexed by the step's rows)
    assert decode_splits(1, 8, 148, 2048) == 32 and decode_splits(1, 8, 148, 13000) == 64
    assert decode_splits(1, 8, 148, 30000) == 128 and decode_splits(2, 8, 148, 30000) == 64
    assert decode_splits(8, 8, 148, 30000) == 16 and decode_splits(1, 8, 148, None, capacity=65536) == 128
    assert decode_splits(1, 8, 148, None, capacity=16384) == 32
    _, _, _, mx, _ = plan_items([1, 300], [30000, 300], group=4, nkv=8, window=None, sm_count=148, rows_per_cta=128,
                                whole_tiles_kernel=True)
    assert mx == 32
    # for the fast tile kernel: 32 tiles x 8 kv heads (less than two CTAs per SM) stay
    # whole; two tiles over a long prefix (a quarter of the SMs at most) are still cut
    _, _, _, mx, cut = plan_items([1024], [1024], group=4, nkv=8, window=None, sm_count=148, rows_per_cta=128,
                                  whole_tiles_kernel=True)
    assert not cut and mx == 1
    _, _, _, mx, cut = plan_items([1024], [1024], group=4, nkv=8, window=None, sm_count=148, rows_per_cta=128)
    assert cut and mx > 1
    _, _, _, mx, cut = plan_items([64], [9000], group=4, nkv=8, window=None, sm_count=148, rows_per_cta=128,
                                  whole_tiles_kernel=True)
    assert cut and mx > 1
    tiles, dec, row_splits, mx, tile_split = plan_items([40, 1], [100, 513], group=4, nkv=8, window=None, sm_count=148)
    # 40 tokens x group 4 fill a 128-row tile: 32 tokens per tile, 2 whole tiles;
    # the decode row: 513 keys -> 16 slices of >= 32 keys, 4 per CTA
    assert sorted((int(i[0]), int(i[1]), int(i[3])) for i in tiles) == [(0, 0, 1), (0, 32, 1)]
    assert not tile_split and mx == 16 and row_splits.tolist() == [1] * 40 + [16]
    assert [(int(i[0]), int(i[2]), int(i[3])) for i in dec] == [(1, 0, 16), (1, 4, 16), (1, 8, 16), (1, 12, 16)]
    tiles, dec, row_splits, mx, _ = plan_items([1] * 64, [2048] * 64, group=4, nkv=8, window=None, sm_count=148)
    assert mx == 4 and len(dec) == 64 and len(tiles) == 0   # a full grid: one CTA of four slices per row
    tiles, dec, row_splits, mx, tile_split = plan_items([5], [900], group=4, nkv=2, window=None, sm_count=148)
    assert tile_split and mx == 7 and len(tiles) == 7       # 15 key tiles -> slices of >= 2 tiles


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(100, 96), (128, 512), (1000, 1536), (4096 + 48, 4096), (200, 12288)])
def test_gemm_skinny(M, N, K):
    """The weight-streaming decode product for every cluster size it may pick, against float64."""
    from openinfer_b200.kernels import linear as lin
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    from openinfer_b200.kernels import lib as klib
    L = klib.load()
    for c in (1, 2, 4, 8):
        if K % (32 * c) or 49152 + 32 * (K // c + 64) + 4096 > 200 * 1024:   # the slice must fit in shared memory
            continue
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
            klib.check(L.oi_gemm_skinny(out.data_ptr(), 1 if out_dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                        x.stride(0), w.data_ptr(), w.stride(0), M, N, K, 0, 0, c,
                                        torch.cuda.current_stream().cuda_stream), "gemm_skinny")
            tol_ = 2e-2 * ref.abs().max().item() if out_dtype == torch.bfloat16 else 2e-4 * ref.abs().max().item()
            err = (out.double() - ref).abs().max().item()
            assert err <= tol_, f"cluster {c} {out_dtype}: max err {err}"


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 512), (3, 100, 72), (16, 4096 + 48, 4096), (17, 300, 1000),
                                   (40, 520, 4096), (100, 384, 2048), (128, 1000, 8192), (8, 200, 12288)])
def test_gemm_stream(M, N, K):
    """The tcgen05 weight-streaming product (weight rows on the M side of the MMA, tokens padded to
    16 / 32 / 64 / 128 by the copy's zero fill) for every number of K slices, against float64."""
    from openinfer_b200.kernels import linear as lin
    from openinfer_b200.kernels import lib as klib
    torch.manual_seed(M * 1000 + N)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    L = klib.load()
    num_kb = -(-K // 64)
    for c in (1, 2, 4, 8):
        if (c - 1) * (-(-num_kb // c)) >= num_kb or (c > 1 and M > 32):   # refused by the entry point
            continue
        for out_dtype in (torch.bfloat16, torch.float32):
            out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
            klib.check(L.oi_gemm_stream(out.data_ptr(), 1 if out_dtype == torch.bfloat16 else 0, out.stride(0), x.data_ptr(),
                                        x.stride(0), w.data_ptr(), w.stride(0), M, N, K, c, 0,
                                        torch.cuda.current_stream().cuda_stream), "gemm_stream")
            tol_ = 2e-2 * ref.abs().max().item() if out_dtype == torch.bfloat16 else 2e-4 * ref.abs().max().item()
            err = (out.double() - ref).abs().max().item()
            assert err <= tol_, f"{c} slices {out_dtype}: max err {err}"
    assert lin.stream_status() == 0, "a bounded wait ran out in the streaming product"
    if M <= lin.DECODE_MAX_ROWS:
        # the dispatcher takes it, and a row does not depend on the other rows
        out = lin.linear(x, w)
        assert (out.double() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
        one = lin.linear(x[M - 1:], w)
        assert torch.equal(one[0], out[M - 1])


@pytest.mark.parametrize("M", [1, 8, 20, 32])
@pytest.mark.parametrize("H,K", [(320, 512), (1024, 2048), (4096, 1024)])
def test_gemm_stream_takes_the_norms_of_a_decode_layer_into_itself(M, H, K):
    """The streaming product's two additions against float64: a product that ends a residual branch adds the
    residual and leaves the next norm's inputs (rows times the norm weight, partial sums of squares per tile and
    K slice); the product behind it scales its rows by rsqrt(mean square + eps). Together: residual add, RMSNorm
    and projection without a norm kernel. Every number of K slices the shape allows; a width that is no multiple
    of the tile (320); gate/up with the activation as the second product."""
    import ctypes
    from openinfer_b200.kernels import lib as klib, linear as lin, native
    L = klib.load()
    torch.manual_seed(M + H)
    eps, off, inter = 1e-5, 0.25, 256
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)                 # the branch's last activations
    w1 = (torch.randn(H, K, device=DEV) * 0.05).to(torch.bfloat16)        # the branch's last projection
    h = torch.randn(M, H, device=DEV).to(torch.bfloat16)                 # the residual stream
    wn = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16)        # the next norm's weight
    w2 = (torch.randn(2 * inter, H, device=DEV) * 0.05).to(torch.bfloat16)   # gate|up in blocks of 64
    stream = torch.cuda.current_stream().cuda_stream
    for c in (1, 2, 4, 8):
        if (c - 1) * (-(-(K // 64) // c)) >= K // 64:
            continue
        h_new = h.clone()
        xs = torch.full((M, H), float("nan"), device=DEV, dtype=torch.bfloat16)
        units = -(-H // 128) * c
        stride = -(-units // 4) * 4 + 4
        ssq = torch.full((32, stride), float("nan"), device=DEV)          # whatever lies beyond the units is not read
        ep = native.StreamEpilogue(residual=h_new.data_ptr(), ld_residual=H, norm_w=wn.data_ptr(), norm_w_bf16=1,
                                   w_offset=off, xs=xs.data_ptr(), ld_xs=H, ssq_out=ssq.data_ptr(), ssq_stride=stride)
        klib.check(L.oi_gemm_stream_fused(h_new.data_ptr(), 1, H, a.data_ptr(), K, w1.data_ptr(), K, M, H, K, c, 0,
                                          ctypes.byref(ep), stream), "gemm_stream_fused")
        want_h = h.double() + a.double() @ w1.double().t()
        assert (h_new.double() - want_h).abs().max().item() <= 2e-2 * want_h.abs().max().item(), f"{c} slices: residual sum"
        hr = h_new.double()                                              # what the kernel rounded is what it normalises
        assert torch.equal(xs, (hr * (off + wn.double())).to(torch.bfloat16)), f"{c} slices: rows times the norm weight"
        got_ssq = ssq[:M, :units].double().sum(1)
        assert torch.allclose(got_ssq, (hr * hr).sum(-1), rtol=1e-5), f"{c} slices: sums of squares"
        assert torch.isnan(ssq[M:]).all() and torch.isnan(ssq[:, units:]).all(), "written outside its rows and units"
        # the product behind it: plain, and gate/up with the activation
        rstd = torch.rsqrt((hr * hr).mean(-1, keepdim=True) + eps)
        for act in (0, 1):
            n_out = inter if act else 2 * inter
            out = torch.full((M, n_out), float("nan"), device=DEV, dtype=torch.bfloat16)
            ep2 = native.StreamEpilogue(ssq_in=ssq.data_ptr(), ssq_units=units, ssq_stride=stride, inv_width=1.0 / H, eps=eps)
            klib.check(L.oi_gemm_stream_fused(out.data_ptr(), 1, n_out, xs.data_ptr(), H, w2.data_ptr(), H, M, 2 * inter, H,
                                              L.oi_stream_slices(2 * inter, H), act, ctypes.byref(ep2), stream), "gemm_stream_fused")
            y = (xs.double() @ w2.double().t()) * rstd
            if act:
                y = y.view(M, -1, 2, 64)
                g, u = y[:, :, 0], y[:, :, 1]
                y = (g / (1 + torch.exp(-g)) * u).reshape(M, inter)
            assert (out.double() - y).abs().max().item() <= 2e-2 * y.abs().max().item(), f"{c} slices, act {act}: scaled product"
    assert lin.stream_status() == 0


def test_gemm_stream_refuses_bad_operands():
    from openinfer_b200.kernels import lib as klib
    L = klib.load()
    x = torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros(4, 128, device=DEV, dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    # two slices of a single k block, 129 rows of x, a cluster for more than 32 rows, a misaligned weight
    for args in [(4, 128, 64, 2), (129, 128, 64, 1), (40, 128, 256, 2)]:
        rc = L.oi_gemm_stream(out.data_ptr(), 1, out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), *args, 0, stream)
        assert rc != 0 and b"gemm_stream" in L.oi_last_error()
    rc = L.oi_gemm_stream(out.data_ptr(), 1, out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr() + 2, w.stride(0), 4, 127, 64, 1, 0, stream)
    assert rc != 0 and b"aligned" in L.oi_last_error()


@pytest.mark.parametrize("M,N,K", [(1, 96, 224), (8, 4096, 12288), (13, 200, 1536)])
def test_gemm_skinny_with_fused_activation(M, N, K):
    from openinfer_b200.kernels import linear as lin
    torch.manual_seed(M + N)
    gu = torch.randn(M, 2 * K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    g, u = gu[:, :K].double(), gu[:, K:].double()       # the reference activation in float64, rounded once like the kernel's
    act = (g / (1.0 + torch.exp(-g)) * u).to(torch.bfloat16)
    ref = act.double() @ w.double().t()
    for fused in (False, True):
        lin.FUSE_SILU_MUL = fused
        try:
            out = lin.linear_silu_mul(gu, w)
        finally:
            lin.FUSE_SILU_MUL = False
        assert (out.double() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item(), f"fused={fused}"


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gate_activation_is_an_argument_of_every_kernel_that_forms_it(act):
    """act(gate) * up against float64 from the formulas, in the four kernels that form it: the stand-alone
    kernel (both dtypes, block layouts), the streaming product, the tcgen05 products (single CTAs and pairs)
    and the skinny product's staging loop."""
    from openinfer_b200.kernels import gemm_tcgen05 as g, linear as lin, ops

    def activation(x):
        if act == "silu":
            return x / (1.0 + torch.exp(-x))
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))

    torch.manual_seed(3)
    K, inter = 256, 512
    for M in (5, 20, 300):
        x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        wg = (torch.randn(inter, K, device=DEV) * 0.1).to(torch.bfloat16)
        wu = (torch.randn(inter, K, device=DEV) * 0.1).to(torch.bfloat16)
        ref = activation(x.double() @ wg.double().t()) * (x.double() @ wu.double().t())
        tol = 2e-2 * ref.abs().max().item()
        w = torch.stack([wg.view(-1, 64, K), wu.view(-1, 64, K)], dim=1).reshape(2 * inter, K).contiguous()
        if M <= 32:
            out = lin.gate_up_silu_mul(x, w, act)
            assert out is not None and (out.double() - ref).abs().max().item() <= tol, f"streaming product, {M} rows"
        for tile in (256, g.PAIR):
            out = torch.full((M, inter), float("nan"), device=DEV, dtype=torch.bfloat16)
            g.gemm_silu_mul(out, x, w, tile, act)
            assert (out.double() - ref).abs().max().item() <= tol, f"tcgen05 product, tile {tile}, {M} rows"
        gu = (x.float() @ w.float().t())                      # [M, 2 inter] in blocks of 64
        for dtype in (torch.float32, torch.bfloat16):
            buf = gu.to(dtype)
            gd = buf.double().view(M, -1, 2, 64)
            want = (activation(gd[:, :, 0]) * gd[:, :, 1]).reshape(M, inter)
            out = torch.full((M, inter), float("nan"), device=DEV, dtype=dtype)
            ops.silu_mul(out, buf, 64, act)
            bound = 1e-5 if dtype == torch.float32 else 1e-2
            assert (out.double() - want).abs().max().item() <= bound * max(1.0, want.abs().max().item()), f"stand-alone {dtype}"
        if M <= 16:
            wd = (torch.randn(96, inter, device=DEV) * 0.05).to(torch.bfloat16)
            buf = gu.to(torch.bfloat16)
            gd = buf.double().view(M, -1, 2, 64)
            a = (activation(gd[:, :, 0]) * gd[:, :, 1]).reshape(M, inter).to(torch.bfloat16)
            want = a.double() @ wd.double().t()
            lin.FUSE_SILU_MUL = True
            try:
                out = lin.linear_silu_mul(buf, wd, 64, act)
            finally:
                lin.FUSE_SILU_MUL = False
            assert (out.double() - want).abs().max().item() <= 2e-2 * want.abs().max().item(), "skinny product"
    assert g.status() == 0 and lin.stream_status() == 0


@pytest.mark.parametrize("M,N,K", [(2048, 4096, 12288), (64, 1024, 25600), (33, 151, 72), (500, 3001, 1024)])
def test_products_of_more_than_32_rows_add_up_in_float32(M, N, K):
    """The dispatcher's product for steps of more than 32 rows (the vendor library called from native code, or the
    package's own tcgen05 kernel where the library has nothing) against float64, with sums of up to 25,600 terms: the
    bound is what float32 accumulation with ONE rounding of the result leaves (half a bfloat16 ulp of the result plus
    a little); partial sums of a split K rounded to bfloat16 would break it. Output in bfloat16 and in float32."""
    from openinfer_b200.kernels import linear as lin
    torch.manual_seed(K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    out = lin.linear(x, w)
    err = (out.double() - ref).abs()
    assert (err <= ref.abs() * 2.0 ** -8 + 1e-3 * ref.abs().max()).all(), f"bfloat16 out: max err {err.max().item()}"
    out32 = lin.linear(x, w, out_dtype=torch.float32)
    err32 = (out32.double() - ref).abs().max().item()
    assert err32 <= 2e-4 * ref.abs().max().item(), f"float32 out: max err {err32}"


@pytest.mark.parametrize("tile_n", [256, 128, 0])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 4096), (300, 520, 1000), (2048, 1024, 512),
                                   (17, 100, 72), (129, 257, 8), (2048, 5120, 192), (600, 1100, 2048), (2048, 2560, 1536)])
def test_gemm_tcgen05(M, N, K, tile_n):
    """The tcgen05 / TMEM / TMA product against float64: whole tiles, ragged edges in M, N and K; tiles of
    one CTA (tile_n columns) and 256 x 256 tiles of a pair of CTAs (0). (2048, 5120, 192) and (2048, 2560, 1536)
    give every pair of CTAs more than one tile, so both accumulators and every stage are used again."""
    from openinfer_b200.kernels import gemm_tcgen05 as g
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    scale = ref.abs().max().item()
    for out_dtype, tol_ in ((torch.bfloat16, 1e-2), (torch.float32, 1e-4)):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
        g.gemm(out, x, w, tile_n)
        assert g.status() == 0, "a bounded wait ran out"
        err = (out.double() - ref).abs().max().item()
        assert err <= tol_ * scale, f"{out_dtype}: max err {err} (scale {scale})"
    # operand rows with a stride wider than K (a view into a larger buffer)
    big = torch.randn(M, K + 16, device=DEV).to(torch.bfloat16)
    out = torch.empty(M, N, device=DEV, dtype=torch.float32)
    g.gemm(out, big[:, :K], w, tile_n)
    assert g.status() == 0
    assert (out.double() - big[:, :K].double() @ w.double().t()).abs().max().item() <= 1e-4 * scale


@pytest.mark.parametrize("tile_n", [256, 0])
@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 384, 200), (2048, 1024, 512), (520, 640, 2048), (2048, 1280, 1536)])
def test_gemm_tcgen05_with_activation_in_the_epilogue(M, I, K, tile_n):
    """silu(x Wg^T) * (x Wu^T) from one kernel, gate and up rows interleaved in blocks of 64."""
    from openinfer_b200.kernels import gemm_tcgen05 as g
    torch.manual_seed(M + I)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    wg = (torch.randn(I, K, device=DEV) * 0.1).to(torch.bfloat16)
    wu = (torch.randn(I, K, device=DEV) * 0.1).to(torch.bfloat16)
    nb = I // g.ACT_BLOCK
    w = torch.stack([wg.view(nb, g.ACT_BLOCK, K), wu.view(nb, g.ACT_BLOCK, K)], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    g.gemm_silu_mul(out, x, w, tile_n)
    assert g.status() == 0
    gg, uu = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    ref = gg / (1 + torch.exp(-gg)) * uu
    assert (out.double() - ref).abs().max().item() <= 1.5e-2 * ref.abs().max().item()


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (8, 192, 520), (16, 12288, 4096), (13, 448, 1000)])
def test_gemm_stream_with_activation(M, I, K):
    """The decode gate/up product with silu(gate) * up formed where the K slices are added up."""
    from openinfer_b200.kernels import gemm_tcgen05 as g
    from openinfer_b200.kernels import lib as klib
    from openinfer_b200.kernels import linear as lin
    torch.manual_seed(M + I)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    wg = (torch.randn(I, K, device=DEV) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(I, K, device=DEV) * 0.05).to(torch.bfloat16)
    nb = I // g.ACT_BLOCK
    w = torch.stack([wg.view(nb, g.ACT_BLOCK, K), wu.view(nb, g.ACT_BLOCK, K)], dim=1).reshape(2 * I, K).contiguous()
    gg, uu = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    ref = gg / (1 + torch.exp(-gg)) * uu
    L = klib.load()
    num_kb = -(-K // 64)
    for c in (1, 2, 4, 8):
        if (c - 1) * (-(-num_kb // c)) >= num_kb:
            continue
        out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
        klib.check(L.oi_gemm_stream(out.data_ptr(), 1, out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                                    M, 2 * I, K, c, 1, torch.cuda.current_stream().cuda_stream), "gemm_stream")
        assert (out.double() - ref).abs().max().item() <= 1.5e-2 * ref.abs().max().item(), f"{c} slices"
    assert lin.stream_status() == 0
    act = lin.gate_up_silu_mul(x, w)
    assert act is not None and (act.double() - ref).abs().max().item() <= 1.5e-2 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_block_layout(dtype):
    from openinfer_b200.kernels import ops
    rows, inter, block = 5, 384, 128
    g = (torch.randn(rows, inter, device=DEV) * 2).to(dtype)
    u = torch.randn(rows, inter, device=DEV).to(dtype)
    gu = torch.stack([g.view(rows, -1, block), u.view(rows, -1, block)], dim=2).reshape(rows, 2 * inter).contiguous()
    out = torch.empty(rows, inter, device=DEV, dtype=dtype)
    ops.silu_mul(out, gu, block)
    ref = g.float() / (1 + torch.exp(-g.float())) * u.float()
    assert torch.allclose(out.float(), ref, **tol(dtype))


@pytest.mark.parametrize("nq,nkv,hd,rot", [(8, 2, 128, 128), (5, 1, 64, 32), (3, 3, 32, 32)])
def test_qk_norm_rope_kv_write_many_tokens(nq, nkv, hd, rot):
    """Prompt-sized launches take the path in which a warp walks over several heads of a token."""
    from openinfer_b200.kernels import ops
    from openinfer_b200.parts.position import RotaryEncoding
    from openinfer_b200.parts.spec import PositionSpec
    torch.manual_seed(hd)
    dtype = torch.bfloat16
    T, P, theta, eps, max_pos = 300, 16, 1e6, 1e-6, 512
    pages = 24
    width = (nq + 2 * nkv) * hd
    qkv = torch.randn(T, width, device=DEV).to(dtype)
    src = qkv.clone().float().cpu()
    positions = torch.randint(0, max_pos, (T,), dtype=torch.int32)
    slots = torch.randperm(pages * P)[:T].to(torch.int32)
    slots[7] = -1
    qw, kw = (1 + 0.1 * torch.randn(hd)).to(dtype), (1 + 0.1 * torch.randn(hd)).to(dtype)
    cos, sin = RotaryEncoding(PositionSpec("rope", rot, theta, max_pos)).rotation_tables(torch.device(DEV))
    cache = torch.zeros(2, pages, P, nkv, hd, device=DEV, dtype=dtype)   # [k/v, pages, P, nkv, hd]
    ops.qk_norm_rope_kv(qkv, nq, nkv, hd, q_norm_w=qw.to(DEV), k_norm_w=kw.to(DEV), eps=eps, weight_offset=0.0,
                        cos=cos, sin=sin, positions=positions.to(DEV), slots=slots.to(DEV), k_cache=cache[0],
                        v_cache=cache[1], page_stride=cache.stride(1), page_size=P)
    q_ref = _rope_ref(src[:, : nq * hd].view(T, nq, hd), positions, rot, theta, qw.float(), eps, 0.0)
    k_ref = _rope_ref(src[:, nq * hd: (nq + nkv) * hd].view(T, nkv, hd), positions, rot, theta, kw.float(), eps, 0.0)
    v_ref = src[:, (nq + nkv) * hd:].view(T, nkv, hd)
    assert torch.allclose(qkv[:, : nq * hd].float().cpu().view(T, nq, hd), q_ref, atol=2e-2, rtol=2e-2)
    flat = cache.float().cpu().view(2, pages * P, nkv, hd)
    ok = slots >= 0
    assert torch.allclose(flat[0][slots[ok].long()], k_ref[ok], atol=2e-2, rtol=2e-2)
    assert torch.equal(flat[1][slots[ok].long()], v_ref[ok])
    untouched = torch.ones(pages * P, dtype=torch.bool)
    untouched[slots[ok].long()] = False
    assert flat[:, untouched].abs().sum() == 0


@pytest.mark.parametrize("nq,nkv,hd,rot,P,norm", [(32, 8, 128, 128, 16, True), (6, 2, 64, 32, 8, True), (4, 1, 32, 32, 16, False),
                                                  (16, 1, 128, 64, 32, True)])
@pytest.mark.parametrize("write_kv", [True, False])
def test_attention_decode_with_norm_rotation_and_cache_write_fused(nq, nkv, hd, rot, P, norm, write_kv):
    """A step of single tokens: the decode kernel takes the raw projection, normalises and rotates q and k
    and stores k and v itself. Same outputs and same cache as the rotation kernel followed by attention."""
    from openinfer_b200.kernels import attention as A
    from openinfer_b200.kernels import ops
    from openinfer_b200.parts.position import RotaryEncoding
    from openinfer_b200.parts.spec import PositionSpec
    torch.manual_seed(nq * 7 + hd)
    kv_lens = [1, 16, 17, 33, 100, 257, 640]
    B = len(kv_lens)
    pages = [-(-kv // P) for kv in kv_lens]
    total = sum(pages) + 3
    perm = torch.randperm(total).tolist()
    bt = torch.zeros(B, max(pages), dtype=torch.int32)
    at = 0
    for b in range(B):
        bt[b, : pages[b]] = torch.tensor(perm[at: at + pages[b]])
        at += pages[b]
    cache0 = (torch.randn(total, 2, P, nkv, hd, device=DEV) * 0.7).to(torch.bfloat16)
    qkv0 = torch.randn(B, (nq + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    cos, sin = RotaryEncoding(PositionSpec("rope", rot, 5000.0, 1024)).rotation_tables(torch.device(DEV))
    qw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=DEV)).to(torch.bfloat16) if norm else None
    positions = torch.tensor([kv - 1 for kv in kv_lens], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(bt[b, (kv - 1) // P]) * P + (kv - 1) % P for b, kv in enumerate(kv_lens)], dtype=torch.int32, device=DEV)
    slots[2] = -1 if not write_kv else slots[2]      # (only meaningful without the write: stays unused)
    scale = 1.0 / math.sqrt(hd)
    results = []
    for fused in (False, True):
        cache, qkv = cache0.clone(), qkv0.clone()
        out = torch.full((B, nq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
        ctx = _FakeCtx([1] * B, kv_lens, P)
        grp = _FakeGroup(bt.to(DEV), kv_lens)
        k_c, v_c = cache[:, 0], cache[:, 1]
        if fused:
            assert A.decode_takes_rope(qkv, ctx, grp, nq, nkv, hd, None, cos, qw, cache.stride(0))   # a grid of one wave
            rope = A.RopeFusion(qw, kw, 1e-6, 0.0, cos, sin, positions, slots, write_kv)
            A.paged_attention(qkv, out, k_c, v_c, cache.stride(0), ctx, grp, nq, nkv, hd, scale, None, rope=rope)
            assert torch.equal(qkv, qkv0), "the fused kernel leaves the projection as it is"
        else:
            ops.qk_norm_rope_kv(qkv, nq, nkv, hd, q_norm_w=qw, k_norm_w=kw, eps=1e-6, weight_offset=0.0, cos=cos, sin=sin,
                                positions=positions, slots=slots, k_cache=k_c, v_cache=v_c, page_stride=cache.stride(0),
                                page_size=P, write_kv=write_kv)
            assert A.attention_mma(qkv[:, : nq * hd], out, k_c, v_c, cache.stride(0), ctx, grp, nq, nkv, hd, scale, None)
        results.append((out.float(), cache.float()))
    (o0, c0), (o1, c1) = results
    assert torch.isfinite(o1).all()
    assert (c0 - c1).abs().max().item() <= 1e-2 * c0.abs().max().item(), "the cache after the step"
    if not write_kv:
        assert torch.equal(c1, cache0.float()), "nothing is stored when the call reads another call's cache"
    assert (o0 - o1).abs().max().item() <= 2e-2, f"outputs differ by {(o0 - o1).abs().max().item()}"


@pytest.mark.parametrize("nq,nkv,hd,P", [(8, 2, 128, 16), (4, 1, 128, 64), (6, 2, 32, 16), (4, 4, 64, 8)])
@pytest.mark.parametrize("rows", [1, 40])
def test_tensor_core_attention_finds_one_far_key_and_respects_the_window(nq, nkv, hd, P, rows):
    """The tuned kernels (decode rows: rows = 1; prompt tiles, tcgen05 where head_dim is 128: rows = 40):
    ONE key among 700 is made to stand out for every query row; the output must be that key's value
    wherever it lies (first key, edges of pages and of 64-key tiles, the last visible key). With a window
    that just excludes it, it must not be seen at all."""
    from openinfer_b200.kernels import attention as A
    torch.manual_seed(hd + rows)
    S = 700
    scale = 1.0 / math.sqrt(hd)
    n_pages = -(-S // P) + 4
    order = torch.randperm(n_pages).tolist()
    bt = torch.tensor([order[: -(-S // P)]], dtype=torch.int32, device=DEV)
    first_row_pos = S - rows
    for far in (0, P - 1, P, 63, 64, 65, 127, 128, 383, 384, first_row_pos - 1, first_row_pos):
        direction = torch.randn(hd)
        direction /= direction.norm()
        # a window of S - 1 - far keys: the last row (position S - 1) just misses `far`, the rows before it see it
        for window in (None, S - 1 - far if far < first_row_pos else None):
            k = torch.randn(S, nkv, hd) * 0.1
            v = torch.randn(S, nkv, hd)
            k[far] = direction * 12.0
            cache = _paged(k, v, P, order, torch.bfloat16, n_pages).to(DEV)
            q = (direction * 12.0 * math.sqrt(hd) / 2).repeat(rows, nq, 1).to(torch.bfloat16)
            qd = q.view(rows, -1).to(DEV)
            out = torch.full((rows, nq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
            ctx = _FakeCtx([rows], [S], P)
            grp = _FakeGroup(bt, [S])
            assert A.attention_mma(qd, out, cache[:, 0, 0], cache[:, 0, 1], cache.stride(0), ctx, grp, nq, nkv, hd, scale, window)
            assert A.tcgen05_status() == 0
            got = out.float().cpu().view(rows, nq, hd)
            want = v[far].to(torch.bfloat16).float()     # [nkv, hd]
            if window is None:
                for r in range(rows):
                    for h in range(nq):
                        assert torch.allclose(got[r, h], want[h // (nq // nkv)], atol=3e-2), f"far key {far}: row {r}, head {h}"
            else:
                # the window of the LAST row ends just after `far`: that row must not see it; row 0 still does
                assert not torch.allclose(got[rows - 1, 0], want[0], atol=0.2), f"key {far} seen outside a window of {window}"
                if rows > 1:
                    assert torch.allclose(got[0, 0], want[0], atol=3e-2), f"key {far} not seen by row 0 inside a window of {window}"


def test_copy_words_between_pinned_host_memory_and_the_device():
    """A step's metadata goes to the device, and the drawn tokens come back, by a kernel that reads or
    writes pinned host memory; token ids that the host does not know yet are put in on the way."""
    from openinfer_b200.kernels import ops
    n, ids_off, src_off, n_ids = 300, 8, 40, 20
    host = torch.arange(n, dtype=torch.int32).pin_memory()
    host[src_off: src_off + n_ids] = -1
    host[src_off + 3] = 2          # id 3 comes from tokens[2], id 7 from tokens[0]
    host[src_off + 7] = 0
    host[src_off + 9] = 99         # outside the tokens: left alone
    tokens = torch.tensor([1000, 1001, 1002], dtype=torch.int32, device=DEV)
    dev = torch.full((n + 5,), -7, dtype=torch.int32, device=DEV)
    ops.copy_words(dev, host, n, ids_off=ids_off, src_off=src_off, n_ids=n_ids, tokens=tokens)
    want = host.clone()
    want[ids_off + 3], want[ids_off + 7] = 1002, 1000
    assert torch.equal(dev[:n].cpu(), want) and bool((dev[n:] == -7).all())
    back = torch.zeros(n, dtype=torch.int32).pin_memory()
    ops.copy_words(back, dev, n)
    torch.cuda.synchronize()
    assert torch.equal(back, want)
    with pytest.raises(Exception):
        ops.copy_words(dev, torch.zeros(n, dtype=torch.int32), n)      # pageable host memory is refused


@pytest.mark.parametrize("vocab", [37, 5000, 151936])
def test_token_logprobs(vocab):
    """log-softmax of a picked token and the k most likely ones, ties to the lowest id
    (pegainfer-sample/src/lib.rs:305-358), for rows listed out of a larger logits tensor."""
    from openinfer_b200.kernels import ops
    torch.manual_seed(vocab)
    logits = torch.randn(6, vocab) * 3
    logits[2, 5] = logits[2, 11] = logits[2].max() + 1.0        # a tie at the top: id 5 comes first
    logits[4] = 0.25                                             # all equal: ids 0, 1, 2, ...
    rows = [4, 0, 2, 2, 5]
    picked = [3, 7, 11, 0, vocab - 1]
    ks = [4, 0, 3, 1, 5]
    lp, vals, ids = ops.token_logprobs(logits.to(DEV), torch.tensor(rows, dtype=torch.int32, device=DEV),
                                       torch.tensor(picked, dtype=torch.int32, device=DEV),
                                       torch.tensor(ks, dtype=torch.int32, device=DEV), 5)
    lp, vals, ids = lp.cpu(), vals.cpu(), ids.cpu()
    ref = torch.log_softmax(logits.double(), dim=-1)
    for i, (r, p, k) in enumerate(zip(rows, picked, ks)):
        assert abs(float(lp[i]) - float(ref[r, p])) < 2e-4
        order = sorted(range(vocab), key=lambda j: (-float(logits[r, j]), j))[:k]
        assert ids[i, :k].tolist() == order, f"row {r}: top-{k} ids"
        assert torch.allclose(vals[i, :k].double(), ref[r, order], atol=2e-4)
        assert (ids[i, k:] == -1).all() and bool(torch.isinf(vals[i, k:]).all())


@pytest.mark.parametrize("nq,nkv,hd", [(4, 2, 128), (4, 1, 64)])
def test_attention_mma_long_contexts(nq, nkv, hd):
    """Thousands of keys: a 1,500-token portion over a 1,500-token prefix (many query tiles, up to 47 key tiles
    each, block-table rounds of the TMA producer), and decode rows at 5,000 and 3,001 keys (32 key slices)."""
    plan = _mma_case(nq, nkv, hd, 16, None, [1500, 1, 1, 300], [3000, 5000, 3001, 300], seed=3)
    assert plan.num_tile_items and plan.num_decode_items
