"""The kernels behind the Givirax parts, each alone against plain float64 arithmetic: the scaled embedding with learned
positions, the 32-bit residual update with its norm, tanh-GELU, the cache write of keys, the router, the experts, and
attention over keys that are also the values (general and tensor-core kernels) with keys made to stand out just inside
and just outside the window, among the kept first positions, and at page borders."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ops():
    from cppvllm_b200.csrc import ops as o
    o.core()
    return o


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [50, 176])
def test_embedding_with_scale_and_learned_positions(ops, dt, D):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(37, D, generator=g).to(dt)
    pos_table = torch.randn(29, D, generator=g).to(dt)
    tokens = torch.tensor([3, 36, 0, 3, 17], dtype=torch.int32)
    positions = torch.tensor([0, 28, 5, 6, 7], dtype=torch.int32)
    out = torch.empty(5, D, device=dev())
    out2 = torch.empty(5, D, device=dev())
    ops.embed_positions(out, table.to(dev()), tokens.to(dev()), positions.to(dev()), 1.75, pos_table.to(dev()), out2)
    ref = table.double()[tokens.long()] * 1.75 + pos_table.double()[positions.long()]
    assert torch.allclose(out.cpu().double(), ref, atol=1e-6, rtol=1e-6) and torch.equal(out, out2)
    ops.embed_positions(out, table.to(dev()), tokens.to(dev()), positions.to(dev()))            # no scale, no positions
    assert torch.equal(out.cpu(), table.float()[tokens.long()])


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [50, 96, 4100])
def test_residual_update_and_norm(ops, dt, D):
    g = torch.Generator().manual_seed(1)
    T = 7
    h0 = torch.randn(T, D, generator=g) * 3
    d1, d2 = torch.randn(T, D, generator=g).to(dt), torch.randn(T, D, generator=g).to(dt)
    rows, vec, w = torch.randn(T, D, generator=g), torch.randn(D, generator=g), torch.rand(D, generator=g) + 0.5
    for use in ((), ("d1",), ("d1", "d2"), ("rows", "vec"), ("d1", "d2", "rows", "vec"), ("vec",)):
        for norm in (False, True):
            if not use and not norm:
                continue
            h = h0.clone().to(dev())
            out = torch.full((T, D), float("nan"), dtype=dt, device=dev()) if norm else None
            deltas = tuple(t.to(dev()) for n, t in (("d1", d1), ("d2", d2)) if n in use)
            ops.resid_update(h, deltas, rows=rows.to(dev()) if "rows" in use else None, vector=vec.to(dev()) if "vec" in use else None,
                             norm_weight=w.to(dev()) if norm else None, eps=1e-3, out=out)
            ref = h0.double()
            if "d1" in use:
                ref = ref + (d1.double() + (d2.double() if "d2" in use else 0))
            if "rows" in use:
                ref = ref + rows.double()
            if "vec" in use:
                ref = ref + vec.double()
            assert torch.allclose(h.cpu().double(), ref, atol=2e-6, rtol=1e-6), use
            if norm:
                n = ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + 1e-3) * w.double()
                tol = 1e-5 if dt == torch.float32 else 1e-2
                assert torch.allclose(out.cpu().double(), n, atol=tol, rtol=tol), use


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gelu_tanh_and_key_rows_into_pages(ops, dt):
    x = torch.linspace(-6, 6, 1001).to(dt).to(dev())
    out = torch.empty_like(x)
    ops.gelu_tanh(out, x)
    z = x.cpu().double()
    ref = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    assert torch.allclose(out.cpu().double(), ref, atol=1e-6 if dt == torch.float32 else 2e-2, rtol=1e-6 if dt == torch.float32 else 1e-2)
    KV, hd, ps, H = 3, 10, 4, 6
    src = torch.randn(5, (H + KV) * hd).to(dt).to(dev())
    pages = torch.zeros(6, KV, ps, hd, dtype=dt, device=dev())
    slots = torch.tensor([9, 2, 23, -1, 8], dtype=torch.int32, device=dev())
    ops.write_rows(pages, src, slots, H * hd, KV, hd, ps)
    ref = torch.zeros_like(pages)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            ref[s // ps, :, s % ps, :] = src[t, H * hd:].view(KV, hd)
    assert torch.equal(pages, ref)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,D", [(8, 2, 48), (3, 1, 50), (4, 4, 64), (40, 33, 96)])
def test_router_top_k_and_renormalised_weights(ops, dt, E, top, D):
    g = torch.Generator().manual_seed(2)
    T = 19
    x = torch.randn(T, D, generator=g).to(dt)
    wr, b = torch.randn(E, D, generator=g), torch.randn(E, generator=g) * 2
    wr[E - 1] = wr[0]                                       # equal rows, equal biases: equal logits, the lower index first
    b[E - 1] = b[0]
    ids = torch.empty(T, top, dtype=torch.int32, device=dev())
    wts = torch.empty(T, top, dtype=torch.float32, device=dev())
    ops.route_topk(ids, wts, x.to(dev()), wr.to(dev()), b.to(dev()))
    z = x.double() @ wr.double().T + b.double()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        got = ids[t].tolist()
        if 0 in got and E - 1 in got:
            assert got.index(0) < got.index(E - 1)
        assert set(got) - {0, E - 1} == set(order) - {0, E - 1} and (0 in got) >= (E - 1 in got)
        zt = z[t][got]
        ref = torch.softmax(zt, 0)
        assert torch.allclose(wts[t].cpu().double(), ref, atol=1e-5) and abs(float(wts[t].sum()) - 1) < 1e-5


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,D,F,T", [(5, 2, 48, 24, 9), (3, 3, 50, 12, 4), (8, 2, 128, 64, 300), (4, 1, 64, 40, 70), (6, 2, 256, 136, 700),
                                         (16, 3, 64, 8, 130)])
def test_experts_against_plain_arithmetic(ops, dt, E, top, D, F, T):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, D, generator=g).to(dt)
    wgu = (torch.randn(E, 2 * F, D, generator=g) * 0.2).to(dt)
    wd = (torch.randn(E, D, F, generator=g) * 0.2).to(dt)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.softmax(torch.randn(T, top, generator=g), -1)
    ref = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            gate, up = wgu[e, :F].double() @ x[t].double(), wgu[e, F:].double() @ x[t].double()
            ref[t] += wts[t, k].double() * (wd[e].double() @ (gate * torch.sigmoid(gate) * up))
    tol = 2e-5 if dt == torch.float32 else 3e-2
    kernels = ["", "rows"] + (["tcgen05"] if dt == torch.bfloat16 and D % 8 == 0 and F % 8 == 0 else [])
    for kernel in kernels:                                   # every path gives the same sums, to rounding
        y = torch.full((T, D), float("nan"), dtype=dt, device=dev())
        ops.routed_experts(y, x.to(dev()), ids.to(dev()), wts.to(dev()), wgu.to(dev()), wd.to(dev()), kernel=kernel)
        ops.check_device_errors(dev())
        assert float((y.cpu().double() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), kernel


def paged_keys(keys, page, order_seed):
    """keys [n, KV, hd] into pages [P, KV, page, hd] in a scrambled order; returns (pages, table)."""
    n, KV, hd = keys.shape
    n_pages = (n + page - 1) // page
    perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(order_seed))[:n_pages]
    pages = torch.full((n_pages + 3, KV, page, hd), float("nan"), dtype=keys.dtype)     # what no token may touch is NaN
    for j in range(n):
        pages[perm[j // page], :, j % page, :] = keys[j]
    return pages, perm.to(torch.int32)


def attention_plain(q, keys, positions, H, KV, hd, scale, window, keep):
    out = torch.zeros(len(positions), H, hd, dtype=torch.float64)
    for t, p in enumerate(positions):
        js = [j for j in range(p + 1) if window <= 0 or p - j < window or j < keep]
        for h in range(H):
            k = keys[js, h // (H // KV)].double()
            s = (k @ q[t, h].double()) * scale
            w = torch.softmax(s, 0)
            out[t, h] = w @ k
    return out


def run_both(ops, q, keys, positions_by_seq, H, KV, hd, page, scale, window, keep, dt, tensor_cores, splits=0):
    """q [T, H, hd]; one request per entry of positions_by_seq (consecutive positions), all reading the same keys."""
    pages, table = paged_keys(keys.to(dt), page, 7)
    S = len(positions_by_seq)
    tables = table.unsqueeze(0).repeat(S, 1).contiguous()
    # pages wholly before a request's window that hold no kept position are given back in the engine: entry -1
    for s, ps_ in enumerate(positions_by_seq):
        lo = max(0, ps_[0] - window + 1) if window > 0 else 0
        for slot in range(lo // page):
            if window > 0 and slot * page >= keep:
                tables[s, slot] = -1
    positions = [p for ps_ in positions_by_seq for p in ps_]
    T = len(positions)
    cu = torch.tensor([0] + list(torch.tensor([len(x) for x in positions_by_seq]).cumsum(0)), dtype=torch.int32)
    seq_of = torch.tensor([s for s, ps_ in enumerate(positions_by_seq) for _ in ps_], dtype=torch.int32)
    pad = torch.zeros(T, KV * hd, dtype=dt)
    packed = torch.cat([q.to(dt).reshape(T, H * hd), pad], dim=1).contiguous().to(dev())   # as a projection leaves it
    out = torch.full((T, H * hd), float("nan"), dtype=dt, device=dev())
    pos_t = torch.tensor(positions, dtype=torch.int32, device=dev())
    if tensor_cores:
        q_lens = [len(x) for x in positions_by_seq]
        scratch = torch.full((ops.attn_keys_scratch_floats(S, KV, hd, max(1, splits)),), float("nan"), device=dev()) if splits > 1 else None
        ops.attn_keys_bf16(out, packed, pages.to(dev()), tables.to(dev()), cu.to(dev()), pos_t, S, ops.attn_keys_tiles(q_lens, H, KV),
                           H, KV, hd, page, scale, window=window, keep_first=keep, all_single=splits > 0, splits=max(1, splits),
                           scratch=scratch)
    else:
        ops.paged_attention_general(out, packed, pages.to(dev()), tables.to(dev()), seq_of.to(dev()), pos_t, H, KV, hd, page, scale,
                                    window=window, num_tokens=T, keep_first=keep, keys_are_values=True)
    ops.check_device_errors(dev())
    return out.float().cpu().view(T, H, hd), positions


CASES = [  # H, KV, hd, page, window, keep
    (6, 3, 96, 32, 45, 5), (6, 2, 64, 16, 70, 3), (3, 1, 16, 16, 9, 2), (8, 8, 128, 64, 130, 70), (5, 5, 32, 16, 64, 0),
    (4, 1, 48, 32, 0, 0), (2, 2, 80, 16, 1, 1), (16, 2, 112, 32, 33, 40)]


@pytest.mark.parametrize("tensor_cores", [False, True])
@pytest.mark.parametrize("H,KV,hd,page,window,keep", CASES)
def test_attention_over_keys_random(ops, H, KV, hd, page, window, keep, tensor_cores):
    dt = torch.bfloat16 if tensor_cores else torch.float32
    g = torch.Generator().manual_seed(hd + window)
    n = 300
    keys = torch.randn(n, KV, hd, generator=g)
    if dt == torch.bfloat16:
        keys = keys.to(dt).float()
    # a prompt portion behind cached tokens, a whole prompt, single decoded tokens near and far, a portion of two tokens
    seqs = [list(range(120, 299)), list(range(0, 150)), [0], [1], [window if window else 5], [299], [200, 201], [63, 64, 65]]
    T = sum(len(s) for s in seqs)
    q = torch.randn(T, H, hd, generator=g)
    if dt == torch.bfloat16:
        q = q.to(dt).float()
    scale = 0.9 / math.sqrt(hd)
    got, positions = run_both(ops, q, keys, seqs, H, KV, hd, page, scale, window, keep, dt, tensor_cores)
    ref = attention_plain(q, keys, positions, H, KV, hd, scale, window, keep)
    tol = 1e-5 if dt == torch.float32 else 2e-2
    assert float((got.double() - ref).abs().max()) <= tol * float(ref.abs().max())


@pytest.mark.parametrize("splits", [1, 2, 8])
@pytest.mark.parametrize("H,KV,hd,page,window,keep", CASES)
def test_attention_of_decoded_tokens_alone(ops, H, KV, hd, page, window, keep, splits):
    """The form for steps in which every request brings one token: positions at the start of a sequence, around the
    window's and the kept tokens' edges, at tile and page borders and far out; one block per (request, kv head) and the
    tiles shared out among 2 and 8 blocks."""
    g = torch.Generator().manual_seed(hd * 3 + window)
    n = 700
    keys = torch.randn(n, KV, hd, generator=g).to(torch.bfloat16).float()
    ps = sorted({0, 1, 2, keep, max(0, keep - 1), 31, 32, 33, 63, 64, 65, window, max(0, window - 1), window + 1, window + keep,
                 255, 256, 300, 511, 699} & set(range(n)))
    seqs = [[p] for p in ps]
    q = torch.randn(len(ps), H, hd, generator=g).to(torch.bfloat16).float()
    scale = 0.9 / math.sqrt(hd)
    got, positions = run_both(ops, q, keys, seqs, H, KV, hd, page, scale, window, keep, torch.bfloat16, True, splits=splits)
    ref = attention_plain(q, keys, positions, H, KV, hd, scale, window, keep)
    assert float((got.double() - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("tensor_cores", [False, True])
@pytest.mark.parametrize("H,KV,hd,page,window,keep", [(6, 3, 96, 32, 45, 5), (6, 2, 64, 16, 70, 3), (2, 1, 32, 16, 64, 17),
                                                      (2, 2, 128, 64, 100, 64)])
def test_a_key_that_stands_out_shows_every_edge(ops, H, KV, hd, page, window, keep, tensor_cores):
    """One key among hundreds is made to dominate (its query match is scaled up): the output is that key while it is
    visible and something else entirely when it is not.  The key is placed just inside and just outside the window, on
    the last kept position and the first one not kept, and on both sides of page borders; the query is a decoded token,
    the last token of a portion, and a token in the middle of a portion."""
    dt = torch.bfloat16 if tensor_cores else torch.float32
    g = torch.Generator().manual_seed(5)
    n = 400
    keys = torch.randn(n, KV, hd, generator=g) * 0.1
    marks = {}
    p = 333
    for name, j in (("window_in", p - window + 1), ("window_out", p - window), ("kept_in", keep - 1), ("kept_out", keep),
                    ("page_border_in", (p - window + 1) // page * page + page), ("self", p)):
        if 0 <= j <= p:
            marks[name] = j
    scale = 1.0
    for name, j in marks.items():
        k2 = keys.clone()
        k2[j] = torch.randn(KV, hd, generator=g)                 # a large, distinct key
        k2[j] = k2[j] / k2[j].norm(dim=-1, keepdim=True) * 6.0
        if dt == torch.bfloat16:
            k2 = k2.to(dt).float()
        sees = (p - j < window) or (j < keep)
        for seqs, t in (([[p]], 0), ([list(range(p - 50, p + 1))], 50), ([list(range(p - 20, p + 30))], 20)):
            T = len(seqs[0])
            q = torch.randn(T, H, hd, generator=g) * 0.1
            for h in range(H):
                q[t, h] = k2[j, h // (H // KV)] * 1.5             # score 54 against the marked key, about 0 elsewhere
            if dt == torch.bfloat16:
                q = q.to(dt).float()
            got, positions = run_both(ops, q, k2, seqs, H, KV, hd, page, scale, window, keep, dt, tensor_cores,
                                      splits=2 if tensor_cores and len(seqs[0]) == 1 else 0)
            assert positions[t] == p
            for h in range(H):
                target = k2[j, h // (H // KV)]
                close = float((got[t, h] - target).abs().max()) < 0.05
                assert close == sees, (name, j, h, len(seqs[0]), float((got[t, h] - target).abs().max()))
            ref = attention_plain(q, k2, positions, H, KV, hd, scale, window, keep)
            assert float((got.double() - ref).abs().max()) <= (1e-5 if dt == torch.float32 else 3e-2) * float(ref.abs().max())
