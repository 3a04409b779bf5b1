"""Per-kernel parity on the GPU, through the C ABI (cudabert_k_* entry points), against the
oracle's functions evaluated in fp32 on the same seeded inputs."""
import math

import numpy as np
import pytest
import torch

from oracle import bert_oracle

pytestmark = pytest.mark.gpu

EPI_BIAS, EPI_GELU, EPI_RESIDUAL, EPI_TANH, EPI_OUT_F32, EPI_COLSCALE, EPI_OUT_F16 = 1, 2, 4, 8, 16, 32, 64
EPI_WSCALE, EPI_IN_F16, EPI_W_FP8 = 128, 256, 512
# what they pass in FP8-weight mode: E4M3 weight bytes widened inside the kernel, per-column scale
ENCODER_LINEAR_FP8 = EPI_BIAS | EPI_OUT_F16 | EPI_IN_F16 | EPI_COLSCALE | EPI_W_FP8
W_CONTAINER_SCALE = 4096.0
# what the encoder's dense layers pass in bf16 mode: fp16 operands and output, weights held scaled
ENCODER_LINEAR = EPI_BIAS | EPI_OUT_F16 | EPI_IN_F16 | EPI_WSCALE

# bf16 has 8 significand bits: one rounding is 2^-9 relative; outputs here see two (input and
# output rounding) on top of fp32 accumulation order differences.
BF16_REL_TOL = 1.0e-2
F16_REL_TOL = 2.0e-3   # fp16: 11 significand bits
FP32_ABS_TOL = 2.0e-4


@pytest.fixture(scope="module")
def pybert():
    from cudabert_b200.cuda_bert import pybert as pb
    torch.backends.cuda.matmul.allow_tf32 = False
    return pb


def _ref_epilogue(acc, flags, bias, resid, colscale):
    if flags & EPI_COLSCALE:
        acc = acc * colscale
    if flags & EPI_WSCALE:
        acc = acc / W_CONTAINER_SCALE
    if flags & EPI_BIAS:
        acc = acc + bias
    if flags & EPI_RESIDUAL:
        acc = acc + resid.float()
    if flags & EPI_GELU:
        acc = bert_oracle.gelu(acc)
    if flags & EPI_TANH:
        acc = torch.tanh(acc)
    return acc


GEMM_SHAPES = [(128, 256, 64), (128, 128, 64), (1, 256, 128), (300, 768, 768), (1000, 2304, 768),
               (515, 3072, 768), (2048, 1024, 4096), (4100, 4096, 1024), (77, 384, 192)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("flags", [0, EPI_BIAS, EPI_BIAS | EPI_GELU, EPI_BIAS | EPI_RESIDUAL,
                                   EPI_BIAS | EPI_TANH | EPI_OUT_F32, EPI_BIAS | EPI_COLSCALE, EPI_BIAS | EPI_OUT_F16,
                                   EPI_BIAS | EPI_GELU | EPI_COLSCALE, EPI_BIAS | EPI_RESIDUAL | EPI_OUT_F32,
                                   ENCODER_LINEAR, ENCODER_LINEAR | EPI_GELU,
                                   EPI_BIAS | EPI_OUT_F16 | EPI_IN_F16 | EPI_COLSCALE,
                                   EPI_BIAS | EPI_GELU | EPI_OUT_F16 | EPI_IN_F16 | EPI_COLSCALE,
                                   EPI_IN_F16 | EPI_OUT_F32])
def test_gemm_tcgen05(pybert, M, N, K, flags):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K + flags)
    in_dt = torch.float16 if flags & EPI_IN_F16 else torch.bfloat16
    A = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(in_dt)
    W = torch.randn(N, K, device="cuda", generator=g) * 0.05
    if flags & EPI_W_FP8:    # E4M3 bytes (values up to +-448), widened to fp16 inside the kernel
        W8 = (W * 2000.0).to(torch.float8_e4m3fn)
        W, Wref = W8.view(torch.uint8), W8.float()
    elif flags & EPI_WSCALE:   # bf16-rounded weights held as fp16 numbers times the container scale
        W = (W.bfloat16().float() * W_CONTAINER_SCALE).half()
        assert torch.equal(W.float() / W_CONTAINER_SCALE, (W.float() / W_CONTAINER_SCALE).bfloat16().float())
    else:
        W = W.to(in_dt)
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    colscale = torch.rand(N, device="cuda", generator=g) + 0.5
    if flags & EPI_W_FP8:
        colscale = (colscale / 2000.0).contiguous()      # undoes the quantisation scale, as the model's per-tensor scale does
    out_f32 = bool(flags & EPI_OUT_F32)
    resid = torch.randn(M, N, device="cuda", generator=g)
    resid = resid if out_f32 else resid.bfloat16()
    odt = torch.float32 if out_f32 else (torch.float16 if flags & EPI_OUT_F16 else torch.bfloat16)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=odt)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = pybert.k_gemm_tcgen05(A.data_ptr(), K, W.data_ptr(), M, N, K, out.data_ptr(), flags, bias.data_ptr(),
                            resid.data_ptr(), colscale.data_ptr(), err.data_ptr())
    assert rc == 0, "k_gemm_tcgen05 rc=%d err=%d" % (rc, int(err.item()))
    if not flags & EPI_W_FP8:
        Wref = W.float()
    ref = _ref_epilogue(A.float() @ Wref.t(), flags, bias, resid, colscale)
    got = out.float()
    assert torch.isfinite(got).all()
    rel = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    tol = F16_REL_TOL if (flags & EPI_IN_F16) and (flags & (EPI_OUT_F16 | EPI_OUT_F32)) else BF16_REL_TOL
    assert rel <= tol, "rel err %.3g" % rel


def test_gemm_bf16_strided_rows(pybert):
    """The pooler reads row b*S of the hidden states: A rows with a stride larger than K."""
    B, S, H = 37, 13, 768
    g = torch.Generator(device="cuda").manual_seed(5)
    hidden = torch.randn(B * S, H, device="cuda", generator=g).bfloat16()
    W = (torch.randn(H, H, device="cuda", generator=g) * 0.05).bfloat16()
    bias = torch.randn(H, device="cuda", generator=g) * 0.1
    out = torch.empty(B, H, device="cuda", dtype=torch.float32)
    rc = pybert.k_gemm_tcgen05(hidden.data_ptr(), S * H, W.data_ptr(), B, H, H, out.data_ptr(),
                            EPI_BIAS | EPI_TANH | EPI_OUT_F32, bias.data_ptr(), None, None, None)
    assert rc == 0
    ref = torch.tanh(hidden.view(B, S, H)[:, 0].float() @ W.float().t() + bias)
    assert (out - ref).abs().max().item() <= 5e-3


@pytest.mark.parametrize("M,N,K", [(8, 768, 768), (1024, 2304, 768), (333, 3072, 768), (130, 1024, 4096)])
@pytest.mark.parametrize("flags", [EPI_BIAS, EPI_BIAS | EPI_GELU, EPI_BIAS | EPI_RESIDUAL, EPI_BIAS | EPI_TANH])
def test_gemm_f32(pybert, M, N, K, flags):
    g = torch.Generator(device="cuda").manual_seed(M + N + K + flags)
    A = torch.randn(M, K, device="cuda", generator=g) * 0.5
    W = torch.randn(K, N, device="cuda", generator=g) * 0.05
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    resid = torch.randn(M, N, device="cuda", generator=g)
    out = torch.full((M, N), float("nan"), device="cuda")
    rc = pybert.k_gemm_f32(A.data_ptr(), K, W.data_ptr(), M, N, K, out.data_ptr(), flags, bias.data_ptr(),
                           resid.data_ptr())
    assert rc == 0
    ref = _ref_epilogue((A.double() @ W.double()).float(), flags, bias, resid, None)
    assert (out - ref).abs().max().item() <= FP32_ABS_TOL


@pytest.mark.parametrize("M,N,K", [(8, 768, 768), (1024, 2304, 768), (333, 3072, 768), (130, 1024, 4096),
                                   (657, 768, 3072), (2000, 4096, 1024)])
@pytest.mark.parametrize("flags", [EPI_BIAS, EPI_BIAS | EPI_GELU, EPI_BIAS | EPI_RESIDUAL, 0])
def test_gemm_f32_on_tensor_cores(pybert, M, N, K, flags):
    """fp32 mode's default GEMM: both operands as three bf16 planes, six cross terms on the tcgen05
    pipeline.  Against float64 it has to be at the level of an fp32 GEMM (within 2e-6 of the sum of
    |a||w|, element by element; two bf16 planes alone would leave 2^-16 = 1.5e-5), not merely within the
    mode's budget; the rows of A span ten binary orders of magnitude."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K + flags)
    A = torch.randn(M, K, device="cuda", generator=g) * torch.exp2(torch.randint(-6, 4, (M, 1), device="cuda",
                                                                                 generator=g).float())
    W = torch.randn(K, N, device="cuda", generator=g) * 0.05
    bias = torch.randn(N, device="cuda", generator=g) * 0.1
    resid = torch.randn(M, N, device="cuda", generator=g)
    out = torch.full((M, N), float("nan"), device="cuda")
    rc = pybert.k_gemm_f32_tensor(A.data_ptr(), K, W.data_ptr(), M, N, K, out.data_ptr(), flags, bias.data_ptr(),
                                  resid.data_ptr())
    assert rc == 0
    exact = A.double() @ W.double()
    ref = _ref_epilogue(exact.float(), flags, bias, resid, None)
    err = (out - ref).abs()
    # element-wise against sum_k |a||w|: the planes drop less than 2^-22 of it, and the tensor core's
    # fp32 accumulator adds its own rounding per 16-product step (up to 1 536 steps); GELU (slope <= 1.13)
    # passes that on and adds the 2.5e-5 of its polynomial
    scale = (A.abs().double() @ W.abs().double()).float()
    bound = 2e-6 * scale + 2e-7 * ref.abs() + 1e-9 + (5e-5 if flags & EPI_GELU else 0.0)
    worst = (err / bound).max().item()
    assert worst <= 1.0, "error is %.2f x the bound" % worst
    if not flags & EPI_GELU:
        plain = (A @ W)          # torch's own fp32 GEMM on the same inputs, for scale
        print("max err %.3g (torch fp32 GEMM: %.3g)" % (err.max().item(), (plain - exact.float()).abs().max().item()))


@pytest.mark.parametrize("M,H,K1,N2,gelu", [(300, 768, 768, 3072, 1), (1000, 1024, 4096, 3072, 0), (77, 1024, 1024, 4096, 1),
                                            (2049, 768, 3072, 2304, 0), (1, 256, 64, 128, 0)])
def test_layernorm_folded_into_its_gemms(pybert, M, H, K1, N2, gelu):
    """The GEMM in front of a LayerNorm writes the sum (fp32), the sum times gamma (fp16) and per-row
    partial statistics; the GEMM behind it normalises in its epilogue:
    LN(s) W + b = rstd (s * gamma) W - rstd mu (gamma W) + (beta W + b).  Against the two layers with
    an explicit LayerNorm in float64 on the same fp16 / bf16 inputs; the rows get offsets and scales so
    that the means are not small against the spread."""
    g = torch.Generator(device="cuda").manual_seed(M + H + K1 + N2)
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g)
    A1 = (rnd(M, K1) * 0.5).half()
    W1 = (rnd(H, K1) * 0.05).bfloat16().float()
    W2 = (rnd(N2, H) * 0.05).bfloat16().float()
    b1, b2 = rnd(H) * 0.1, rnd(N2) * 0.1
    res = rnd(M, H) * torch.exp2(torch.randint(-2, 3, (M, 1), device="cuda", generator=g).float()) + rnd(M, 1)
    gamma, beta = 1.0 + 0.3 * rnd(H), 0.2 * rnd(H)
    hold = lambda w: (w * W_CONTAINER_SCALE).half().contiguous()      # the encoder's weight container
    s_out = torch.full((M, H), float("nan"), device="cuda")
    out = torch.full((M, N2), float("nan"), device="cuda", dtype=torch.float16)
    W1h, W2h, res = hold(W1), hold(W2), res.contiguous()
    rc = pybert.k_gemm_ln_folded(A1.data_ptr(), W1h.data_ptr(), b1.data_ptr(), res.data_ptr(), gamma.data_ptr(),
                                 beta.data_ptr(), W2h.data_ptr(), b2.data_ptr(), M, H, K1, N2, gelu, s_out.data_ptr(),
                                 out.data_ptr())
    assert rc == 0
    s = A1.double() @ W1.double().t() + b1.double() + res.double()
    # fp32 accumulation in the tensor core: within 2e-6 of sum |a||w|, element by element
    s_bound = 2e-6 * (A1.double().abs() @ W1.double().abs().t()) + 1e-6 * s.abs() + 1e-6
    assert ((s_out.double() - s).abs() / s_bound).max().item() <= 1.0
    ln = bert_oracle.layer_norm(s, gamma.double(), beta.double())
    ref = ln @ W2.double().t() + b2.double()
    if gelu:
        ref = bert_oracle.gelu(ref)
    # the operand s * gamma is rounded to fp16 (2^-11 relative per element) and so is the output
    scale = ((ln.abs() + (s.mean(-1, keepdim=True) / s.std(-1, keepdim=True)).abs()) @ W2.double().abs().t())
    err = (out.double() - ref).abs()
    bound = 2.0 ** -10 * scale / (H ** 0.5) * 4 + 2.0 ** -10 * ref.abs() + 1e-3
    assert (err / bound).max().item() <= 1.0, "max err %.3g" % err.max().item()
    assert torch.isfinite(out.float()).all()


def _attention_ref(qkv, mask, B, S, heads):
    # float64: in fp32 a row whose keys are all masked loses score bits to the -10000 offset
    H = heads * 64
    q, k, v = [t.view(B, S, heads, 64).permute(0, 2, 1, 3).double() for t in qkv.view(B * S, 3, H).unbind(1)]
    scores = q @ k.transpose(-1, -2) / math.sqrt(64)
    if mask is not None:
        scores = scores + (1.0 - mask.view(B, 1, 1, S).double()) * -10000.0
    ctx = torch.softmax(scores, -1) @ v
    return ctx.permute(0, 2, 1, 3).reshape(B * S, H).float()


def _mask(B, S, mode, g):
    if mode == "none":
        return None
    lens = torch.randint(1, S + 1, (B,), device="cuda", generator=g)
    m = (torch.arange(S, device="cuda")[None, :] < lens[:, None]).int()
    if mode == "full":
        m[:] = 1
    if mode == "holes":
        m = m * (torch.rand(B, S, device="cuda", generator=g) > 0.3).int()
        m[:, 0] = 1
    if mode == "zero_row":
        m[0, :] = 0
    return m.contiguous()


@pytest.mark.parametrize("bf16", [3, 2, 1, 0])
@pytest.mark.parametrize("B,S,heads", [(2, 128, 12), (3, 200, 16), (1, 512, 16), (4, 17, 12), (2, 1, 12), (5, 64, 16),
                                       (2, 65, 12), (3, 129, 16), (2, 300, 12)])
@pytest.mark.parametrize("mode", ["prefix", "none", "holes", "zero_row", "full"])
def test_attention(pybert, bf16, B, S, heads, mode):
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + S + heads)
    H = heads * 64
    qkv = torch.randn(B * S, 3 * H, device="cuda", generator=g)
    mask = _mask(B, S, mode, g)
    x = qkv.half() if bf16 else qkv      # the 16-bit kernels take fp16 Q, K, V and write fp16
    ctx = torch.full((B * S, H), float("nan"), device="cuda", dtype=x.dtype)
    rc = pybert.k_attention(bf16, x.data_ptr(), None if mask is None else mask.data_ptr(), ctx.data_ptr(), B, S, heads)
    if bf16 == 3 and S > 256:
        assert rc != 0      # the persistent kernel holds two sequences' keys, values and queries: S <= 256
        return
    assert rc == 0
    ref = _attention_ref(x.float(), mask, B, S, heads)
    got = ctx.float()
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item()
    # 16-bit kernels: probabilities and the output are rounded to fp16 (2^-11 relative, values up to ~4)
    assert err <= (4e-3 if bf16 else 1e-4), "max abs err %.3g" % err


@pytest.mark.parametrize("B,S,heads,mode", [(64, 200, 16, "prefix"), (300, 64, 12, "prefix"), (40, 256, 16, "holes"),
                                            (33, 130, 16, "zero_row"), (2500, 16, 12, "prefix"), (1025, 33, 16, "holes")])
def test_attention_persistent_matches_per_item_kernel(pybert, B, S, heads, mode):
    """Many more items than SMs, ragged lengths: the persistent kernel hands items and query blocks
    out dynamically, and every block must come out exactly as the one-CTA-per-item kernel computes
    it (the arithmetic is shared), whatever warp took it and in whichever buffer."""
    g = torch.Generator(device="cuda").manual_seed(B + S)
    H = heads * 64
    x = torch.randn(B * S, 3 * H, device="cuda", generator=g).half()
    mask = _mask(B, S, mode, g)
    out = []
    for kernel in (1, 3, 3):
        ctx = torch.full((B * S, H), float("nan"), device="cuda", dtype=torch.float16)
        assert pybert.k_attention(kernel, x.data_ptr(), mask.data_ptr(), ctx.data_ptr(), B, S, heads) == 0
        out.append(ctx)
    assert torch.isfinite(out[0].float()).all()
    assert torch.equal(out[0], out[1]) and torch.equal(out[1], out[2])


@pytest.mark.parametrize("kernel", [1, 2, 3])
@pytest.mark.parametrize("B,S,heads,mode", [(37, 200, 16, "prefix"), (300, 64, 12, "holes"), (9, 256, 16, "zero_row"),
                                            (5, 512, 16, "full"), (64, 17, 12, "none")])
def test_attention_first_query_only(pybert, kernel, B, S, heads, mode):
    """The last layer of a pooler-only pass asks every bf16 attention kernel for the first query of
    each sequence alone, written to row b: the same bits as row b * S of a full run of that kernel."""
    if kernel == 3 and S > 256:
        pytest.skip("the persistent kernel holds sequences of up to 256 tokens")
    g = torch.Generator(device="cuda").manual_seed(B * 31 + S)
    H = heads * 64
    x = torch.randn(B * S, 3 * H, device="cuda", generator=g).half()
    mask = _mask(B, S, mode, g)
    mptr = None if mask is None else mask.data_ptr()
    full = torch.full((B * S, H), float("nan"), device="cuda", dtype=torch.float16)
    first = torch.full((B, H), float("nan"), device="cuda", dtype=torch.float16)
    assert pybert.k_attention(kernel, x.data_ptr(), mptr, full.data_ptr(), B, S, heads) == 0
    assert pybert.k_attention(kernel + 16, x.data_ptr(), mptr, first.data_ptr(), B, S, heads) == 0
    assert torch.isfinite(first.float()).all()
    assert torch.equal(first, full.view(B, S, H)[:, 0])


@pytest.mark.parametrize("kernel", [2, 1, 3, 0])
@pytest.mark.parametrize("B,S,heads,mode", [(37, 200, 16, "prefix"), (300, 64, 12, "prefix"), (300, 64, 12, "holes"),
                                            (9, 256, 16, "zero_row"), (5, 512, 16, "prefix"), (64, 17, 12, "none"),
                                            (700, 8, 12, "prefix"), (3, 130, 16, "full"), (128, 128, 12, "holes")])
def test_attention_packed_rows(pybert, kernel, B, S, heads, mode):
    """A forward pass keeps only the valid rows, back to back.  Every attention kernel must give a
    row the same bits in that layout as with one padded block of S rows per sequence; for the
    tcgen05 kernel this is the case where a tile of 128 query rows holds rows of several sequences
    (up to 128 of them) and walks the key blocks of each."""
    if kernel == 3 and S > 256:
        pytest.skip("the persistent kernel holds sequences of up to 256 tokens")
    g = torch.Generator(device="cuda").manual_seed(B * 17 + S)
    H = heads * 64
    x = torch.randn(B * S, 3 * H, device="cuda", generator=g)
    x = x.half() if kernel else x
    mask = _mask(B, S, mode, g)
    mptr = None if mask is None else mask.data_ptr()
    if mask is None:
        lens = torch.full((B,), S, dtype=torch.long)
    else:
        pos = torch.arange(1, S + 1, device="cuda")[None, :]
        lens = (mask.long() * pos).max(dim=1).values.cpu()
        lens[lens == 0] = S      # no valid key: the sequence keeps all its rows
    rows = torch.cat([torch.arange(b * S, b * S + int(lens[b])) for b in range(B)]).cuda()
    padded = torch.full((B * S, H), float("nan"), device="cuda", dtype=x.dtype)
    assert pybert.k_attention(kernel, x.data_ptr(), mptr, padded.data_ptr(), B, S, heads) == 0
    xp = torch.zeros_like(x)
    xp[: rows.numel()] = x[rows]
    packed = torch.full((B * S, H), float("nan"), device="cuda", dtype=x.dtype)
    assert pybert.k_attention(kernel + 32, xp.data_ptr(), mptr, packed.data_ptr(), B, S, heads) == 0
    got = packed[: rows.numel()]
    assert torch.isfinite(got.float()).all()
    assert torch.equal(got, padded[rows])
    assert torch.isnan(packed[rows.numel():].float()).all()      # nothing is written beyond the packed rows


@pytest.mark.parametrize("seed", range(24))
def test_attention_packed_tiles_random_shapes(pybert, seed):
    """Random batch sizes, padded lengths and length distributions (many one-row sequences, a few long
    ones, holes, rows without valid key): the tcgen05 kernel on packed rows, whichever way it cuts its
    tiles for that length, gives every valid row the bits it gives it in the padded layout, and stays
    within the 16-bit tolerance of the float64 reference."""
    rng = np.random.default_rng(1000 + seed)
    S = int(rng.choice([5, 24, 64, 80, 100, 130, 160, 200, 300, 400, 512]))
    B = int(rng.integers(1, max(2, min(600, 40000 // S))))
    heads = int(rng.choice([12, 16]))
    H = heads * 64
    style = seed % 4
    if style == 0:
        lens = rng.integers(1, S + 1, B)
    elif style == 1:
        lens = np.where(rng.random(B) < 0.8, rng.integers(1, 4, B), rng.integers(1, S + 1, B))
    elif style == 2:
        lens = np.full(B, S)
    else:
        lens = rng.integers(max(1, S // 2), S + 1, B)
    mask = (np.arange(S)[None, :] < lens[:, None]).astype(np.int32)
    if seed % 3 == 0:                                       # holes below the last valid key
        holes = rng.random((B, S)) < 0.2
        holes[:, 0] = False
        holes[np.arange(B), lens - 1] = False
        mask = mask * (~holes)
    if seed % 5 == 0:
        mask[rng.integers(0, B)] = 0                        # a row without valid key keeps all S rows
    lens = np.where(mask.any(1), S - np.argmax(mask[:, ::-1], axis=1), S)
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(B * S, 3 * H, device="cuda", generator=g).half()
    m = torch.from_numpy(np.ascontiguousarray(mask)).cuda()
    rows = torch.cat([torch.arange(b * S, b * S + int(lens[b])) for b in range(B)]).cuda()
    padded = torch.full((B * S, H), float("nan"), device="cuda", dtype=torch.float16)
    assert pybert.k_attention(2, x.data_ptr(), m.data_ptr(), padded.data_ptr(), B, S, heads) == 0
    xp = torch.zeros_like(x)
    xp[: rows.numel()] = x[rows]
    packed = torch.full((B * S, H), float("nan"), device="cuda", dtype=torch.float16)
    assert pybert.k_attention(2 + 32, xp.data_ptr(), m.data_ptr(), packed.data_ptr(), B, S, heads) == 0
    assert torch.equal(packed[: rows.numel()], padded[rows]), "B %d S %d heads %d" % (B, S, heads)
    assert torch.isnan(packed[rows.numel():].float()).all()
    ref = _attention_ref(x.float(), m, B, S, heads)
    assert (padded.float()[rows] - ref[rows]).abs().max().item() <= 4e-3


@pytest.mark.parametrize("bf16", [1, 0])
@pytest.mark.parametrize("H", [768, 1024])
def test_embed_layernorm_and_layernorm(pybert, bf16, H):
    g = torch.Generator(device="cuda").manual_seed(H + bf16)
    B, S, vocab = 5, 37, 4000
    T = B * S
    dt = torch.float16 if bf16 else torch.float32   # the 16-bit output of the row kernels is fp16
    word = torch.randn(vocab, H, device="cuda", generator=g) * 0.02
    pos = torch.randn(512, H, device="cuda", generator=g) * 0.02
    typ = torch.randn(2, H, device="cuda", generator=g) * 0.02
    gamma = 1 + torch.randn(H, device="cuda", generator=g) * 0.1
    beta = torch.randn(H, device="cuda", generator=g) * 0.1
    ids = torch.randint(0, vocab, (T,), device="cuda", generator=g, dtype=torch.int32)
    seg = torch.randint(0, 2, (T,), device="cuda", generator=g, dtype=torch.int32)
    out = torch.empty(T, H, device="cuda", dtype=dt)
    out32 = torch.empty(T, H, device="cuda", dtype=torch.float32)
    rc = pybert.k_embed_layernorm(bf16, ids.data_ptr(), seg.data_ptr(), word.data_ptr(), pos.data_ptr(),
                                  typ.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                  out32.data_ptr(), T, S, H, vocab)
    assert rc == 0
    p = torch.arange(T, device="cuda") % S
    e = word[ids.long()] + pos[p] + typ[seg.long()]
    ref = bert_oracle.layer_norm(e, gamma, beta)
    tol = 4e-3 if bf16 else 2e-5   # fp16 rounding of values up to ~6
    assert (out.float() - ref).abs().max().item() <= tol
    assert (out32 - ref).abs().max().item() <= 2e-5

    x = torch.randn(T, H, device="cuda", generator=g)
    res = torch.randn(T, H, device="cuda", generator=g)
    out2 = torch.empty(T, H, device="cuda", dtype=dt)
    out2_32 = torch.empty(T, H, device="cuda", dtype=torch.float32)
    for in_f16 in (0, 1):
        xin = x.half() if in_f16 else x
        for r in (None, res):
            assert pybert.k_layernorm(bf16, in_f16, xin.data_ptr(), None if r is None else r.data_ptr(),
                                      gamma.data_ptr(), beta.data_ptr(), out2.data_ptr(), out2_32.data_ptr(), T, H) == 0
            ref2 = bert_oracle.layer_norm(xin.float() + (0 if r is None else r), gamma, beta)
            assert (out2.float() - ref2).abs().max().item() <= tol
            assert (out2_32 - ref2).abs().max().item() <= 2e-5
    assert pybert.k_layernorm(bf16, 0, x.data_ptr(), None, gamma.data_ptr(), beta.data_ptr(), out2.data_ptr(), None,
                              T, H) == 0

    # an out-of-range id is clamped and reported, it never reads outside the table
    ids[3] = vocab + 5
    rc = pybert.k_embed_layernorm(bf16, ids.data_ptr(), seg.data_ptr(), word.data_ptr(), pos.data_ptr(),
                                  typ.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), None, T, S, H,
                                  vocab)
    assert rc == 5
