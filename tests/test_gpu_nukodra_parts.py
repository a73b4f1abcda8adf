"""Nukodra's new kernels alone on the GPU, each against the plain implementation's function for the same
mechanism (float64): the residual streams' connections, the norm over a whole projection with the rotation, the
causal convolution with its carried inputs in portions (also through both forms of the kernel), the gated norm
in parts.  (Attention over wide rows and the heads' small matrices are in ``test_gpu_nukodra.py``; the
state-space memories run through the whole-model tests of every cutting.)"""

from __future__ import annotations

import pytest
import torch

import plain_nukodra as plain

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops("cuda:0")


def dev(t, dtype=None):
    return t.to(device="cuda:0", dtype=dtype or t.dtype).contiguous()


@pytest.mark.parametrize("streams,tokens,width", [(1, 3, 40), (2, 1, 64), (3, 37, 100), (8, 5, 24)])
def test_stream_connections(ops, streams, tokens, width):
    gen = torch.Generator().manual_seed(streams * 100 + tokens)
    x = torch.randn(tokens, width, generator=gen)
    X = ops.streams_spread(dev(x), streams)
    assert X.shape == (streams, tokens, width) and bool((X.cpu() == x[None]).all())
    X = dev(torch.randn(streams, tokens, width, generator=gen))
    a, b, a2 = (torch.randn(streams, generator=gen) for _ in range(3))
    M = torch.eye(streams) + 0.3 * torch.randn(streams, streams, generator=gen)
    y = torch.randn(tokens, width, generator=gen)
    before = X.double().cpu()
    u, zeros = ops.streams_read(X, dev(a), want_zeros=True)
    assert torch.allclose(u.double().cpu(), plain.streams_read(before, a.double()), atol=1e-5)
    assert bool((zeros == 0).all())
    # the write alone, then the write that also reads for the next sublayer: the same streams
    X2 = X.clone()
    ops.streams_write(X, dev(M), dev(b), dev(y))
    want = plain.streams_write(before, M.double(), b.double(), y.double())       # mix is indexed [from, to]
    assert torch.allclose(X.double().cpu(), want, atol=1e-5)
    u2, zeros2 = ops.streams_write(X2, dev(M), dev(b), dev(y), next_read=dev(a2))
    assert torch.equal(X2, X) and bool((zeros2 == 0).all())
    assert torch.allclose(u2.double().cpu(), plain.streams_read(want, a2.double()), atol=1e-5)
    assert torch.allclose(ops.streams_sum(X).double().cpu(), want.sum(0), atol=1e-5)
    if streams > 1:                                                              # [from, to], not [to, from]
        assert not torch.allclose(want, plain.streams_write(before, M.double().T, b.double(), y.double()), atol=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,d,dv,rot,norm", [(4, 2, 16, 8, 8, True), (3, 3, 24, 24, 24, True),
                                                           (2, 1, 40, 16, 0, True), (6, 2, 32, 32, 16, False)])
def test_norm_over_the_whole_projection_and_rotation(ops, dtype, heads, kv_heads, d, dv, rot, norm):
    """Rows [pad | q | k | v]: one norm over all of q and one over all of k, then the first `rot` features of each
    head turned; positions near and far (angles in 32-bit), a padding row that stays as it is."""
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(heads * d + rot)
    positions = torch.tensor([0, 1, 2, 77, 5000, 70001, -1], dtype=torch.int32)
    n = positions.numel()
    q_off, k_off, v_off = 8, 8 + heads * d, 8 + (heads + kv_heads) * d
    proj = torch.randn(n, v_off + kv_heads * dv, generator=gen).to(t)
    q_gain, k_gain = 1 + 0.3 * torch.randn(heads * d, generator=gen), 1 + 0.3 * torch.randn(kv_heads * d, generator=gen)
    base, eps = 500.0, 1e-3
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float()
    from mini_gpt_inference_b200.cache.storage import PagedKVView

    pt = 4
    cache = PagedKVView(dev(torch.full((5, kv_heads, pt, d), float("nan")), t), dev(torch.full((5, kv_heads, pt, dv), float("nan")), t),
                        0, pt, None, True)
    slots = torch.tensor([13, 2, 7, 0, 19, 8, -1], dtype=torch.int32)            # flat cache rows: page * pt + row
    got = dev(proj.clone())
    ops.qk_norm_rotary(got, heads, kv_heads, d, dv, q_off, k_off, v_off, norm, eps, rot, dev(freq) if rot else None, cache,
                       dev(slots), dev(positions), q_gain=dev(q_gain) if norm else None, k_gain=dev(k_gain) if norm else None)
    got = got.double().cpu()
    x = proj.double()
    live = positions >= 0
    q, k = x[:, q_off:k_off], x[:, k_off:v_off]
    if norm:
        q, k = plain.rms_norm(q, q_gain.double(), eps), plain.rms_norm(k, k_gain.double(), eps)
    # angles are 32-bit numbers by design (position * frequency, rounded): at position 70,001 that rounding alone
    # moves an angle by some 4e-3, so the plain rotation runs in 32-bit here, after the norm in 64-bit
    q = plain.rotate(q.float().view(n, heads, d), positions.clamp(min=0), rot, base).reshape(n, -1).double()
    tol = 5e-5 if dtype == "float32" else 2e-2
    assert torch.allclose(got[live, q_off:k_off], q[live], atol=tol, rtol=tol)
    assert torch.equal(got[~live], x[~live])                                     # the padding row
    k = plain.rotate(k.float().view(n, kv_heads, d), positions.clamp(min=0), rot, base).double()
    k_rows = cache.k_pages.double().cpu().permute(0, 2, 1, 3).reshape(-1, kv_heads, d)      # [flat row, head, d]
    v_rows = cache.v_pages.double().cpu().permute(0, 2, 1, 3).reshape(-1, kv_heads, dv)
    for i in range(n - 1):
        assert torch.allclose(k_rows[slots[i]], k[i], atol=tol, rtol=tol), f"keys of token {i}"
        assert torch.equal(v_rows[slots[i]], x[i, v_off:].view(kv_heads, dv)), f"values of token {i}"
    written = torch.zeros(5 * pt, dtype=torch.bool)
    written[slots[:-1].long()] = True
    assert bool(torch.isnan(k_rows[~written]).all()) and bool(torch.isnan(v_rows[~written]).all())
    assert torch.equal(got[:, :q_off], x[:, :q_off]) and torch.equal(got[:, v_off:], x[:, v_off:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channels,taps,x_off", [(24, 4, 8), (40, 2, 0), (13, 5, 3), (16, 1, 16), (200, 4, 48)])
def test_causal_convolution_in_portions(ops, dtype, channels, taps, x_off):
    """Two requests, their sequences cut into steps of unequal portions (one token, two, many: more than 64 tokens
    a step and fewer, so both forms of the vector kernel run where the sizes allow 16-byte loads), slots that start
    filled with NaN; against the convolution of each whole sequence."""
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(channels * taps)
    lengths = [150, 61]
    ld = x_off + channels + 8
    xs = [torch.randn(n, ld, generator=gen).to(t) for n in lengths]
    w = torch.randn(channels, taps, generator=gen) / taps ** 0.5
    bias = 0.3 * torch.randn(channels, generator=gen)
    state = dev(torch.full((3, (taps - 1) * channels + 8), float("nan")))
    slots = [2, 0]
    cuts = [[1, 2, 90, 3, 1, 53], [2, 1, 50, 1, 7]]
    got = [[] for _ in lengths]
    done = [0, 0]

    class Ctx:
        pass

    for step in range(max(len(c) for c in cuts)):
        entries = [(r, cuts[r][step]) for r in range(2) if step < len(cuts[r])]
        rows = torch.cat([xs[r][done[r]: done[r] + n] for r, n in entries])
        ctx = Ctx()
        to = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda:0")
        ctx.token_request = to([i for i, (_, n) in enumerate(entries) for _ in range(n)])
        ctx.positions = to([done[r] + j for r, n in entries for j in range(n)])
        ctx.req_q_start = to([sum(n for _, n in entries[:i]) for i in range(len(entries))])
        ctx.req_q_len = to([n for _, n in entries])
        ctx.req_ctx_before = to([done[r] for r, _ in entries])
        ctx.req_state_slot = to([slots[r] for r, _ in entries])
        x = dev(rows)
        out = ops.causal_conv_silu(ctx, x, x_off, channels, dev(w), dev(bias), state)
        ops.conv_state_update(ctx, x, x_off, channels, taps, state)
        at = 0
        for r, n in entries:
            got[r].append(out[at: at + n].double().cpu())
            at += n
            done[r] += n
    tol = 1e-5 if dtype == "float32" else 2e-2
    for r, n in enumerate(lengths):
        assert done[r] == n
        want = plain.silu(plain.causal_conv(xs[r][:, x_off: x_off + channels].double(), w.double(), bias.double()))
        assert torch.allclose(torch.cat(got[r]), want, atol=tol, rtol=tol), f"request {r}"
    assert bool(torch.isnan(state[1]).all())                                     # the unused slot was not touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,parts", [(64, 1), (96, 3), (40, 5), (256, 2)])
def test_gated_norm_in_parts(ops, dtype, width, parts):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(width + parts)
    n, eps = 9, 1e-3
    o = torch.randn(n, width, generator=gen) * torch.linspace(0.1, 5.0, width)    # parts of unequal size
    z = torch.randn(n, width + 8, generator=gen).to(t)
    gain = 1 + 0.3 * torch.randn(width, generator=gen)
    positions = torch.tensor([0, 1, 2, 3, -1, 5, 6, 7, 8], dtype=torch.int32)
    got = ops.gated_group_norm(dev(o), dev(z)[:, :width], dev(gain), parts, eps, t, positions=dev(positions)).double().cpu()
    gated = (o.double() * plain.silu(z[:, :width].double())).view(n, parts, width // parts)
    want = (plain.rms_norm(gated, None, eps).reshape(n, width) * gain.double())
    live = positions >= 0
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert torch.allclose(got[live], want[live], atol=tol, rtol=tol)
    assert bool((got[~live] == 0).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,q_dim,rot,rank", [(3, 24, 8, 40), (1, 16, 16, 16), (5, 10, 6, 20), (2, 128, 64, 256)])
def test_latent_rows_and_turned_query_parts(ops, dtype, heads, q_dim, rot, rank):
    """Rows [pad | q (heads x (q_dim + rot)) | low (rank + rot)]: the cache row is [norm(low[:rank]) * gain | turned
    low[rank:]]; the queries' turned parts land behind `rank` free numbers per head; a padding row writes nothing."""
    from mini_gpt_inference_b200.cache.storage import PagedKVView

    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(heads * rank + rot)
    positions = torch.tensor([0, 3, 1, 900, -1, 33000], dtype=torch.int32)
    slots = torch.tensor([5, 0, 11, 6, -1, 2], dtype=torch.int32)
    n = positions.numel()
    q_off = 8
    low_off = q_off + heads * (q_dim + rot)
    proj = torch.randn(n, low_off + rank + rot, generator=gen).to(t)
    gain = 1 + 0.3 * torch.randn(rank, generator=gen)
    base, eps, pt = 300.0, 1e-3, 4
    freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float()
    pages = dev(torch.full((3, 1, pt, rank + rot), float("nan")), t)
    cache = PagedKVView(pages, pages, 0, pt, None, True, values_in_keys=True)
    q = ops.latent_prepare(dev(proj), heads, q_off, q_dim, rot, low_off, rank, dev(gain), eps, dev(freq), cache, dev(slots),
                           dev(positions)).double().cpu().view(n, heads, rank + rot)
    x = proj.double()
    live = positions >= 0
    pos = positions.clamp(min=0)
    tol = 5e-5 if dtype == "float32" else 2e-2
    # (the plain rotation in 32-bit: angles are 32-bit numbers by design)
    q_rot = plain.rotate(x[:, q_off:low_off].float().view(n, heads, q_dim + rot)[..., q_dim:], pos, rot, base).double()
    assert torch.allclose(q[live][..., rank:], q_rot[live], atol=tol, rtol=tol)
    latent = plain.rms_norm(x[:, low_off: low_off + rank], gain.double(), eps)
    shared = plain.rotate(x[:, low_off + rank:].float().view(n, 1, rot), pos, rot, base).double().view(n, rot)
    rows = pages.double().cpu().view(-1, rank + rot)
    for i in range(n):
        if live[i]:
            assert torch.allclose(rows[slots[i]], torch.cat([latent[i], shared[i]]), atol=tol, rtol=tol), f"token {i}"
    written = torch.zeros(3 * pt, dtype=torch.bool)
    written[slots[live].long()] = True
    assert bool(torch.isnan(rows[~written]).all())
    # a layer that reads another layer's rows prepares its queries and stores nothing
    pages.fill_(float("nan"))
    reader = PagedKVView(pages, pages, 0, pt, None, False, values_in_keys=True)
    q2 = ops.latent_prepare(dev(proj), heads, q_off, q_dim, rot, low_off, rank, None, eps, dev(freq), reader, dev(slots),
                            dev(positions)).double().cpu().view(n, heads, rank + rot)
    assert torch.equal(q2[live][..., rank:], q[live][..., rank:]) and bool(torch.isnan(pages).all())
