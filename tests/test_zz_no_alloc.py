"""cudabert_k_attention_noalloc: the attention kernel for callers that cannot allocate device
memory (code running inside another framework's allocator or memory pool, or in a process whose
device memory is already fully handed out).  Its scratch is a fixed array inside the library, so
this test checks that it returns what the allocating entry point returns, on two consecutive
calls that reuse that array with different batch sizes, and that it refuses batches the array
cannot hold.  The file name keeps it last in collection order."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, S, heads, bf16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    H = heads * 64
    qkv = torch.randn(B * S, 3 * H, device="cuda", generator=g)
    qkv = qkv.half() if bf16 else qkv
    lens = torch.randint(1, S + 1, (B,), device="cuda", generator=g)
    mask = (torch.arange(S, device="cuda")[None, :] < lens[:, None]).int().contiguous()
    return qkv, mask


@pytest.mark.parametrize("bf16", [1, 0])
def test_noalloc_matches_allocating_entry_point(bf16):
    from cudabert_b200.cuda_bert import pybert
    # two calls in a row: the second uses fewer rows than the first left in the shared scratch
    for seed, B, S, heads in ((11, 9, 150, 16), (12, 4, 77, 12)):
        qkv, mask = _case(seed, B, S, heads, bf16)
        H = heads * 64
        ref = torch.full((B * S, H), float("nan"), device="cuda", dtype=qkv.dtype)
        got = torch.full((B * S, H), float("nan"), device="cuda", dtype=qkv.dtype)
        assert pybert.k_attention(bf16, qkv.data_ptr(), mask.data_ptr(), ref.data_ptr(), B, S, heads) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert pybert.k_attention_noalloc(bf16, qkv.data_ptr(), mask.data_ptr(), got.data_ptr(), B, S, heads) == 0
        if not (seed == 11):   # the very first call may load the kernel's module; later calls must not take memory
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert torch.isfinite(got.float()).all()
        # same kernels on the same inputs: the tolerance of the attention tests is far from needed
        tol = 4e-3 if bf16 else 1e-4
        assert (got.float() - ref.float()).abs().max().item() <= tol
        assert torch.equal(got, ref)
    # mask == NULL (all keys valid) also goes through the scratch
    qkv, _ = _case(13, 3, 40, 12, bf16)
    ref = torch.empty(3 * 40, 768, device="cuda", dtype=qkv.dtype)
    got = torch.empty_like(ref)
    assert pybert.k_attention(bf16, qkv.data_ptr(), None, ref.data_ptr(), 3, 40, 12) == 0
    assert pybert.k_attention_noalloc(bf16, qkv.data_ptr(), None, got.data_ptr(), 3, 40, 12) == 0
    assert torch.equal(got, ref)


def test_noalloc_rejects_batches_beyond_its_scratch():
    from cudabert_b200.cuda_bert import pybert
    qkv = torch.zeros(8, 3 * 768, device="cuda", dtype=torch.float16)
    out = torch.zeros(8, 768, device="cuda", dtype=torch.float16)
    rc = pybert.k_attention_noalloc(1, qkv.data_ptr(), None, out.data_ptr(), pybert.NOALLOC_MAX_BATCH + 1, 1, 12)
    assert rc == 6
    assert "CUDABERT_NOALLOC_MAX_BATCH" in pybert.last_error(None)


def test_noalloc_first_query_only_stays_inside_a_batch_sized_output():
    """Kernel 1 + 16 writes one row per sequence: the [B, H] output is followed by a guard region
    that must come back untouched, and the rows equal row b * S of a full run."""
    from cudabert_b200.cuda_bert import pybert
    B, S, heads = 7, 90, 12
    H = heads * 64
    qkv, mask = _case(21, B, S, heads, 1)
    full = torch.empty(B * S, H, device="cuda", dtype=torch.float16)
    assert pybert.k_attention_noalloc(1, qkv.data_ptr(), mask.data_ptr(), full.data_ptr(), B, S, heads) == 0
    buf = torch.full((B + 64, H), 777.0, device="cuda", dtype=torch.float16)   # rows [B, B + 64): guard
    assert pybert.k_attention_noalloc(17, qkv.data_ptr(), mask.data_ptr(), buf.data_ptr(), B, S, heads) == 0
    assert torch.equal(buf[:B], full.view(B, S, H)[:, 0])
    assert bool((buf[B:] == 777.0).all())


@pytest.mark.parametrize("kernel", [2, 3, 18, 16, 5])
def test_noalloc_refuses_kernels_it_cannot_serve(kernel):
    """The tcgen05 and persistent kernels need more scratch than the built-in array holds, and
    "+ 16" needs a 16-bit kernel: refused before anything is launched, with a message."""
    from cudabert_b200.cuda_bert import pybert
    qkv = torch.zeros(64, 3 * 768, device="cuda", dtype=torch.float16)
    out = torch.full((64, 768), 5.0, device="cuda", dtype=torch.float16)
    assert pybert.k_attention_noalloc(kernel, qkv.data_ptr(), None, out.data_ptr(), 2, 32, 12) == 1
    assert "cudabert_k_attention_noalloc" in pybert.last_error(None)
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())
    # a sequence length beyond the kernels' limit is an argument error too, with its own message
    assert pybert.k_attention_noalloc(1, qkv.data_ptr(), None, out.data_ptr(), 1, 513, 12) == 1
    assert "512" in pybert.last_error(None)
