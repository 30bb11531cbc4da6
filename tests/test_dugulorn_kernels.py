"""The kernels that Dugulorn brought, each alone against the plain functions of tests/plain_dugulorn.py (float64): the norm
behind a sublayer, bias and activation, the gated group norm, what stands around latent attention (norms, rotation, cache
write, query assembly, the per-head gate), attention over keys whose leading elements are the value (one key made to
dominate: far away, at page borders, the token's own, read by a decoded token, by the last token of a portion and from the
middle of one), and the two recurrences with their convolutions, continued across portions of every size through state slots
that held something else before."""
import math

import pytest
import torch

import plain_dugulorn as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _ops():
    from cppvllm_b200.csrc import ops
    return ops


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def _dev(t, dtype=None):
    return t.to(DEV, dtype if dtype is not None else t.dtype).contiguous()


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _close(got, ref, tol):
    got, ref = got.detach().cpu().to(F64), ref.to(F64)
    err = float((got - ref).abs().max()) / max(1.0, float(ref.abs().max()))
    assert err <= tol, f"error {err:.3e} of scale beyond {tol:.1e}"


TOLS = {torch.float32: 2e-6, torch.bfloat16: 1.2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [50, 256, 1030])
def test_norm_behind_a_sublayer(dtype, D):
    ops = _ops()
    T = 7
    y = _rand(T, D, seed=1, scale=3.0).to(dtype)
    h0, w, b = _rand(T, D, seed=2), _rand(D, seed=3, scale=0.3), _rand(D, seed=4)
    for bias in (None, b):
        for acc in (True, False):
            h = _dev(h0.clone())
            copy = torch.empty(T, D, dtype=dtype, device=DEV)
            ops.norm_add(h, _dev(y), _dev(1.0 + w), 1e-5, bias=_dev(bias) if bias is not None else None, accumulate=acc, copy=copy)
            yy = y.to(F64) + (bias.to(F64) if bias is not None else 0.0)
            ref = (h0.to(F64) if acc else 0.0) + plain.norm_around_zero(yy, w.to(F64), 1e-5)
            _close(h, ref, 2e-6)
            _close(copy, ref, TOLS[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_and_squared_relu(dtype):
    ops = _ops()
    x, b = _rand(5, 37, seed=5).to(dtype), _rand(37, seed=6)
    out = torch.empty(5, 37, dtype=dtype, device=DEV)
    ops.bias_act(out, _dev(x), _dev(b), "relu2")
    _close(out, torch.relu(x.to(F64) + b.to(F64)) ** 2, TOLS[dtype])
    ops.bias_act(out, _dev(x), None, "none")
    assert torch.equal(out.cpu(), x)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups,G", [(1, 14), (4, 20), (3, 33), (2, 64)])
def test_gated_norm_over_groups(dtype, groups, G):
    ops = _ops()
    T = 6
    o, w = _rand(T, groups * G, seed=7, scale=5.0), 1.0 + _rand(G, seed=8, scale=0.3)
    packed = _rand(T, 9 + groups * G, seed=9).to(dtype)                   # the gate sits inside a wider row
    out = torch.empty(T, groups * G, dtype=dtype, device=DEV)
    dp = _dev(packed)
    ops.gated_norm(out, _dev(o), dp[:, 9:], _dev(w), groups, 1e-4)
    ref = plain.norm_plain(o.to(F64).reshape(T, groups, G), w.to(F64), 1e-4) * plain.logistic(packed[:, 9:].to(F64)).reshape(T, groups, G)
    _close(out, ref.reshape(T, -1), TOLS[dtype])


ROT = {"dims": 6, "base": 50.0, "scaling": {"factor": 5.0, "original": 16, "fast": 4.0, "slow": 1.0}}


def _tables(rot, n):
    freq, mag = plain.rotation_frequencies(rot)
    ang = torch.arange(n, dtype=F64)[:, None] * freq[None, :]
    return _dev((torch.cos(ang) * mag).float()), _dev((torch.sin(ang) * mag).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_norms_rotation_cache_write_query_assembly_and_gate(dtype):
    ops = _ops()
    T, q_rank, R, dr, H, dn, dv, page = 9, 10, 12, 8, 3, 5, 7, 4          # 6 of the 8 positional elements turn
    cos, sin = _tables(ROT, 40)
    packed = _rand(T, q_rank + R + dr + H, seed=11, scale=2.0).to(dtype)
    wq, wk = 1.0 + _rand(q_rank, seed=12, scale=0.3), 1.0 + _rand(R, seed=13, scale=0.3)
    positions = [20, 21, 22, 0, 1, 2, 3, 4, 39]
    slots = [13, 14, 15, 4, 5, 6, 7, 0, 9]
    pages = torch.zeros(5, page, R + dr, dtype=dtype, device=DEV)
    cq = torch.empty(T, q_rank, dtype=dtype, device=DEV)
    dp = _dev(packed)
    ops.latent_prep(dp, cq, 0, q_rank, _dev(wq), pages, q_rank, R, dr, 6, _dev(wk), cos, sin, _i32(positions), _i32(slots), 1e-5)
    p64 = packed.to(F64)
    pos = torch.tensor(positions)
    _close(cq, plain.norm_plain(p64[:, :q_rank], wq.to(F64), 1e-5), TOLS[dtype])
    entries = pages.reshape(-1, R + dr)[torch.tensor(slots, device=DEV)]
    _close(entries[:, :R], plain.norm_plain(p64[:, q_rank:q_rank + R], wk.to(F64), 1e-5), TOLS[dtype])
    _close(entries[:, R:], plain.rotate(p64[:, q_rank + R:q_rank + R + dr], pos, ROT), TOLS[dtype])
    untouched = [s for s in range(20) if s not in slots]
    assert float(pages.reshape(-1, R + dr)[torch.tensor(untouched, device=DEV)].abs().max()) == 0.0
    # without a cache to write (a layer that reads another layer's): only the query latent
    ops.latent_prep(dp, cq, 0, q_rank, _dev(wq), None, 0, R, dr, 6, None, None, None, _i32(positions), None, 1e-5)

    q = _rand(T, H * (dn + dr), seed=14).to(dtype)
    q_abs = _rand(H, T, R, seed=15).to(dtype)
    q_out = torch.empty(T, H * (R + dr), dtype=dtype, device=DEV)
    ops.latent_q_assemble(q_out, _dev(q_abs), _dev(q), H, dn, R, dr, 6, cos, sin, _i32(positions))
    got = q_out.reshape(T, H, R + dr)
    assert torch.equal(got[:, :, :R].cpu(), q_abs.transpose(0, 1))
    _close(got[:, :, R:], plain.rotate(q.to(F64).reshape(T, H, dn + dr)[:, :, dn:], pos, ROT), TOLS[dtype])

    o = _rand(H, T, dv, seed=16).to(dtype)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    ops.head_gate(out, _dev(o), dp[:, q_rank + R + dr:], H, dv)
    ref = o.to(F64).transpose(0, 1) * plain.logistic(p64[:, q_rank + R + dr:])[:, :, None]
    _close(out, ref.reshape(T, -1), TOLS[dtype])


def _attention_case(dtype, H, R, dr, page, kernel, seed):
    """Two requests in one step over shuffled pages: a prompt portion of 70 tokens behind 130 cached ones, and a decoded token
    at position 150.  Chosen queries are tied to one key each, so that exactly that key must be found."""
    ops = _ops()
    HD = R + dr
    lens = [200, 151]
    q_of = [list(range(130, 200)), [150]]
    n_pages = sum((n + page - 1) // page for n in lens) + 3
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    keys = [_rand(n, HD, seed=seed + 1 + i) for i, n in enumerate(lens)]
    keys = [k / k.norm(dim=-1, keepdim=True) * math.sqrt(HD) for k in keys]      # equal lengths: no other key scores higher than the one pointed at
    T = sum(len(x) for x in q_of)
    q = _rand(T, H, HD, seed=seed + 9)
    # (request, row within the step's tokens of that request, head, key position): the query points at that key, strongly
    picks = [(0, 0, 0, 0), (0, 69, 1 % H, 199), (0, 35, 2 % H, page - 1), (0, 36, 0, page), (0, 10, H - 1, 127), (0, 11, 0, 128),
             (0, 69, 0, 3), (1, 0, 0, 150), (1, 0, 1 % H, 0), (1, 0, H - 1, 2 * page - 1), (1, 0, 2 % H, 2 * page)]
    base = [0, 70]
    picks = list({(r, row, h): (r, row, h, j) for r, row, h, j in reversed(picks)}.values())      # one key per (row, head)
    for r, row, h, j in picks:
        q[base[r] + row, h] = keys[r][j] * (100.0 / float(keys[r][j].norm() ** 2)) / 0.25
    pages = torch.full((n_pages, page, HD), float("nan"), dtype=dtype)      # what nobody owns holds NaN
    W = max((n + page - 1) // page for n in lens)
    tables = torch.full((2, W), -1, dtype=torch.int32)
    nxt = 0
    for r, n in enumerate(lens):
        for i in range((n + page - 1) // page):
            pg = order[nxt]; nxt += 1
            tables[r, i] = pg
            chunk = keys[r][i * page:(i + 1) * page].to(dtype)
            pages[pg, :chunk.shape[0]] = chunk
            if chunk.shape[0] < page:
                pages[pg, chunk.shape[0]:] = 1e4 if dtype == torch.bfloat16 else 1e30       # behind the last key: large but finite
    positions = q_of[0] + q_of[1]
    seq_of = [0] * 70 + [1]
    out = torch.empty(T, H * R, dtype=dtype, device=DEV)
    qd = _dev(q.reshape(T, H * HD), dtype)
    if kernel == "general":
        ops.paged_attention_general(out, qd, _dev(pages), _dev(tables), _i32(seq_of), _i32(positions), H, 1, HD, page, 0.25,
                                    num_tokens=T, keys_are_values=True, value_dim=R)
    else:
        ops.attn_keys_bf16(out, qd, _dev(pages), _dev(tables), _i32([0, 70, 71]), _i32(positions), 2, ops.attn_keys_tiles([70, 1], H, 1),
                           H, 1, HD, page, 0.25, value_dim=R)
    ops.check_device_errors(torch.device(DEV))
    got = out.cpu().to(F64).reshape(T, H, R)
    qr = q.to(dtype).to(F64)
    worst = 0.0
    for r in range(2):
        kk = keys[r].to(dtype).to(F64)
        for row, p in enumerate(q_of[r]):
            s = (qr[base[r] + row] @ kk[:p + 1].T) * 0.25                    # [H, p + 1]
            ref = torch.softmax(s, dim=-1) @ kk[:p + 1, :R]
            worst = max(worst, float((got[base[r] + row] - ref).abs().max()))
    found = 0
    for r, row, h, j in picks:                                                # the pointed-at key is what comes out
        kk = keys[r].to(dtype).to(F64)
        p = q_of[r][row]
        weight = torch.softmax((qr[base[r] + row, h] @ kk[:p + 1].T) * 0.25, dim=-1)[j]
        if float(weight) > 0.99:                                              # (with few elements another key may lie as close)
            found += 1
            ref = kk[j, :R]
            assert float((got[base[r] + row, h] - ref).abs().max()) < 0.05 * float(ref.abs().max()) + 0.02, (r, row, h, j)
    assert found >= len(picks) - 1
    assert worst < (1e-5 if dtype == torch.float32 else 3e-2), worst


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,dr,page", [(3, 12, 8, 16), (2, 72, 24, 32), (5, 7, 3, 64)])
def test_attention_over_keys_whose_leading_elements_are_the_value_general(dtype, H, R, dr, page):
    _attention_case(dtype, H, R, dr, page, "general", 100 + H)


@pytest.mark.parametrize("H,R,dr,page", [(4, 48, 16, 32), (8, 80, 16, 32), (20, 32, 32, 16), (3, 16, 16, 64), (2, 96, 32, 32)])
def test_attention_over_keys_whose_leading_elements_are_the_value_tensor_cores(H, R, dr, page):
    _attention_case(torch.bfloat16, H, R, dr, page, "tensor", 200 + H)


@pytest.mark.parametrize("H", [8, 20, 32])
def test_tensor_core_decode_form_with_a_narrower_value(H):
    """Every request brings one token: the kernel for decoded tokens, alone and with the keys shared out among blocks; more
    than 16 heads on the one stored entry go in groups."""
    ops = _ops()
    R, dr, page, HD = 80, 16, 32, 96
    groups = min(n for n in range(1, H + 1) if H % n == 0 and H // n <= 16)
    lens = [700, 33, 1, 257]
    keys = [_rand(n, HD, seed=300 + i) for i, n in enumerate(lens)]
    q = _rand(4, H, HD, seed=310)
    q[0, H - 1] = keys[0][5] * 8.0                   # a far key for one head
    q[3, 0] = keys[3][256] * 8.0                     # the token's own key, first in its page
    W = (max(lens) + page - 1) // page
    n_pages = sum((n + page - 1) // page for n in lens)
    pages = torch.zeros(n_pages + 1, page, HD, dtype=torch.bfloat16)
    tables = torch.full((4, W), -1, dtype=torch.int32)
    pg = n_pages
    for r, n in enumerate(lens):                      # pages handed out from the top down
        for i in range((n + page - 1) // page):
            pg -= 1
            tables[r, i] = pg
            chunk = keys[r][i * page:(i + 1) * page].to(torch.bfloat16)
            pages[pg, :chunk.shape[0]] = chunk
    ref = []
    for r, n in enumerate(lens):
        kk = keys[r].to(torch.bfloat16).to(F64)
        s = (q[r].to(torch.bfloat16).to(F64) @ kk.T) * 0.1
        ref.append(torch.softmax(s, dim=-1) @ kk[:, :R])
    ref = torch.stack(ref)
    for splits in (1, 4):
        out = torch.empty(4, H * R, dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attn_keys_scratch_floats(4, groups, HD, splits), dtype=torch.float32, device=DEV) if splits > 1 else None
        ops.attn_keys_bf16(out, _dev(q.reshape(4, H * HD), torch.bfloat16), _dev(pages), _dev(tables), _i32([0, 1, 2, 3, 4]),
                           _i32([n - 1 for n in lens]), 4, 4, H, groups, HD, page, 0.1, all_single=True, splits=splits, scratch=scratch,
                           value_dim=R, kv_heads_in_pages=1)
        _close(out.reshape(4, H, R), ref, 2e-2)


# ---- recurrences ------------------------------------------------------------------------------------------------------

CUTS = [[1], [2], [5, 1, 1], [17, 2, 16, 1, 33], [70]]


def _steps(lengths_per_request):
    """Interleave several requests' portion lists into steps: step i holds the i-th portion of every request that has one."""
    n = max(len(c) for c in lengths_per_request)
    return [[(r, c[i]) for r, c in enumerate(lengths_per_request) if i < len(c)] for i in range(n)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv", [(2, 10, 7), (1, 64, 64), (2, 130, 5), (3, 33, 50), (2, 128, 36), (1, 256, 16)])
def test_lightning_scan_continues_across_portions_and_slots(dtype, H, dk, dv):
    ops = _ops()
    decays = [1.0, 0.5, 0.97][:H]
    W = 2 * H * dk + H * dv + 3
    reqs = [_rand(sum(c), W, seed=400 + i).to(dtype) for i, c in enumerate(CUTS)]
    state = torch.full((4, H * dk * dv + 5), 7.0, dtype=torch.float32, device=DEV)        # slots hold something else
    slot_of = [2, 0, 3, 1, 2]                                                              # the last request uses slot 2 again
    got = [[] for _ in CUTS]
    at = [0] * len(CUTS)
    # requests 0..3 side by side, then request 4 in the slot that request 0 has left
    for group in ([0, 1, 2, 3], [4]):
        for r in group:
            state[slot_of[r], :H * dk * dv].zero_()
        for step in _steps([CUTS[r] for r in group]):
            rows, cu, slots = [], [0], []
            for gi, n in step:
                r = group[gi]
                rows.append(reqs[r][at[r]:at[r] + n]); at[r] += n
                cu.append(cu[-1] + n); slots.append(slot_of[r])
            packed = _dev(torch.cat(rows))
            n_rows = packed.shape[0]
            out = torch.empty(n_rows, H * dv, dtype=torch.float32, device=DEV)
            qf, kf = (torch.empty(n_rows, H * dk, dtype=torch.float32, device=DEV) for _ in range(2))
            vf = torch.empty(n_rows, H * dv, dtype=torch.float32, device=DEV)
            ops.lightning_prep(qf, kf, vf, packed, 3, 3 + H * dk, 3 + 2 * H * dk)
            ops.lightning_scan(out, qf, kf, vf, state, _dev(torch.tensor(decays)), _i32(cu), _i32(slots), len(step), H, dk, dv)
            for i, (gi, n) in enumerate(step):
                got[group[gi]].append(out[cu[i]:cu[i + 1]].cpu())
    ops.check_device_errors(torch.device(DEV))
    for r, x in enumerate(reqs):
        x = x.to(F64)
        T = x.shape[0]
        q = plain.silu(x[:, 3:3 + H * dk]).reshape(T, H, dk)
        k = plain.silu(x[:, 3 + H * dk:3 + 2 * H * dk]).reshape(T, H, dk)
        v = plain.silu(x[:, 3 + 2 * H * dk:3 + 2 * H * dk + H * dv]).reshape(T, H, dv)
        _close(torch.cat(got[r]).reshape(T, H, dv), plain.lightning_rule(q, k, v, decays), 3e-5)
    assert float(state[:, H * dk * dv:].min()) == 7.0                                      # nothing behind the matrices was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 12, 20, 3), (2, 1, 64, 40, 4), (3, 3, 40, 33, 1), (2, 2, 16, 64, 2), (1, 1, 5, 3, 6)])
def test_delta_rule_with_convolutions_continues_across_portions_and_slots(dtype, H, G, dk, dv, taps):
    ops = _ops()
    C = 2 * G * dk + H * dv
    mat = H * dk * dv
    conv_w = _rand(C, taps, seed=500, scale=0.6)
    dt_bias, a_log = _rand(H * dk, seed=501), _rand(H, seed=502) - 2.0
    reqs = [(_rand(sum(c), 2 + C, seed=510 + i).to(dtype), _rand(sum(c), H * dk, seed=520 + i), _rand(sum(c), H, seed=530 + i))
            for i, c in enumerate(CUTS)]
    state = torch.full((4, mat + (taps - 1) * C), 7.0, dtype=torch.float32, device=DEV)
    slot_of = [2, 0, 3, 1, 2]
    got = [[] for _ in CUTS]
    at = [0] * len(CUTS)
    f32 = dict(dtype=torch.float32, device=DEV)
    for group in ([0, 1, 2, 3], [4]):
        for r in group:
            state[slot_of[r]].zero_()
        for step in _steps([CUTS[r] for r in group]):
            rows, arows, brows, cu, slots, seq_of = [], [], [], [0], [], []
            for i, (gi, n) in enumerate(step):
                r = group[gi]
                x, a, b = reqs[r]
                rows.append(x[at[r]:at[r] + n]); arows.append(a[at[r]:at[r] + n]); brows.append(b[at[r]:at[r] + n]); at[r] += n
                cu.append(cu[-1] + n); slots.append(slot_of[r]); seq_of += [i] * n
            packed, T = _dev(torch.cat(rows)), cu[-1]
            qn, kn = torch.empty(T, G * dk, **f32), torch.empty(T, G * dk, **f32)
            vv, gg, bb = torch.empty(T, H * dv, **f32), torch.empty(T, H * dk, **f32), torch.empty(T, H, **f32)
            ops.delta_prep(qn, kn, vv, gg, bb, packed, 2, _dev(conv_w), _dev(torch.cat(arows)), _dev(dt_bias), _dev(a_log),
                           _dev(torch.cat(brows)), state, mat, _i32(seq_of), _i32(cu), _i32(slots), H, G, dk, dv)
            ops.conv_history(state, mat, packed, 2, C, taps, _i32(cu), _i32(slots), len(step))
            out = torch.empty(T, H * dv, **f32)
            ops.delta_scan(out, qn, kn, vv, gg, bb, state, _i32(cu), _i32(slots), len(step), H, G, dk, dv)
            for i, (gi, n) in enumerate(step):
                got[group[gi]].append(out[cu[i]:cu[i + 1]].cpu())
    ops.check_device_errors(torch.device(DEV))
    for r, (x, a, b) in enumerate(reqs):
        T = x.shape[0]
        y = plain.silu(plain.causal_conv(x[:, 2:].to(F64), conv_w.to(F64)))
        q = plain.unit_vectors(y[:, :G * dk].reshape(T, G, dk)) * dk ** -0.5
        k = plain.unit_vectors(y[:, G * dk:2 * G * dk].reshape(T, G, dk))
        v = y[:, 2 * G * dk:].reshape(T, H, dv)
        g = torch.exp(-torch.exp(a_log.to(F64))[None, :, None] * plain.softplus(a.to(F64) + dt_bias.to(F64)).reshape(T, H, dk))
        _close(torch.cat(got[r]).reshape(T, H, dv), plain.delta_rule(q, k, v, g, plain.logistic(b.to(F64))), 3e-5)
