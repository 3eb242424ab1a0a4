"""Host-side contract of the operator, on CPU: the checks that run before any launch, the `Flash64` and SDPA
signatures, mode resolution. Mirrors the reference's launcher tests that need no GPU
(tests/test_flash64_guard.py:29-172 monkeypatches `Flash64._run`; tests/test_kernels.py:346-392 rejects arguments)."""

from __future__ import annotations

import importlib

import pytest
import torch

import fastforks_b200 as ff
from fastforks_b200.flash64 import Flash64, check_flash64

attn_mod = importlib.import_module("fastforks_b200.attention")


def test_cpu_tensors_are_rejected_not_computed() -> None:
    q = torch.zeros(1, 2, 5, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):
        ff.attention(q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        ff.scaled_dot_product_attention(q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        Flash64()(q, q, q, 0.125)


@pytest.mark.parametrize(
    ("shape", "dtype", "word"),
    [((1, 2, 5, 32), torch.float16, "head dim"), ((1, 2, 5, 64), torch.float32, "float16"), ((2, 5, 64), torch.float16, "4-D")],
)
def test_check_operands_messages(shape: tuple, dtype: torch.dtype, word: str) -> None:
    q = torch.zeros(shape, dtype=dtype)
    with pytest.raises(ValueError, match=word):
        attn_mod.check_operands(q, q, q)


def test_flash64_signature_and_variants() -> None:
    assert ff.FLASH_VARIANTS == ("hh", "fh", "ff")
    with pytest.raises(ValueError, match="variant"):
        Flash64("xx")
    f = Flash64("fh", probe=3)
    assert (f.variant, f.probe, f.window) == ("fh", 3, 3)
    with pytest.raises(ValueError, match="variant"):
        Flash64._run("zz", *(torch.zeros(1, 1, 1, 64),) * 3, 1.0)  # noqa: SLF001


def test_flash64_run_is_the_single_choke_point(monkeypatch: pytest.MonkeyPatch) -> None:
    """Like the reference's guard tests, a patched `_run` sees every call with (variant, q, k, v, scale)."""
    calls = []

    def fake(variant: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
        calls.append((variant, q.shape, scale))
        return torch.zeros_like(q)

    monkeypatch.setattr(Flash64, "_run", staticmethod(fake))
    q = torch.zeros(2, 7, 3, 64, dtype=torch.float16)
    out = Flash64("ff")(q, q, q, 0.5)
    assert calls == [("ff", q.shape, 0.5)]
    assert out.shape == q.shape


def test_check_flash64_needs_same_shapes(monkeypatch: pytest.MonkeyPatch) -> None:
    monkeypatch.setattr(attn_mod, "check_operands", lambda *a, **k: None)
    import fastforks_b200.flash64 as f64

    monkeypatch.setattr(f64, "check_operands", lambda *a, **k: None)
    q = torch.zeros(1, 5, 2, 64, dtype=torch.float16)
    k = torch.zeros(1, 6, 2, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="self-attention only"):
        check_flash64(q, k, k)


def test_sdpa_rejects_dropout_and_causal() -> None:
    q = torch.zeros(1, 2, 5, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="dropout"):
        ff.scaled_dot_product_attention(q, q, q, dropout_p=0.1)
    with pytest.raises(ValueError, match="causal"):
        ff.scaled_dot_product_attention(q, q, q, is_causal=True)


def test_strides_and_sizes_of_both_layouts() -> None:
    packed = torch.zeros(2, 9, 3, 4, 64, dtype=torch.float16)  # [B, N, 3, H, 64]
    q = packed.unbind(2)[0]
    assert attn_mod._sizes(q, "bnhd") == (2, 9, 4)  # noqa: SLF001
    assert attn_mod._strides(q, "bnhd") == (9 * 3 * 4 * 64, 3 * 4 * 64, 64)  # noqa: SLF001
    qs = packed.permute(2, 0, 3, 1, 4)[0]  # [B, H, N, 64] view, as in _vit_kernels
    assert attn_mod._sizes(qs, "bhnd") == (2, 9, 4)  # noqa: SLF001
    assert attn_mod._strides(qs, "bhnd") == (9 * 3 * 4 * 64, 3 * 4 * 64, 64)  # noqa: SLF001


def test_bias_view_broadcasts_without_copy() -> None:
    q = torch.zeros(2, 3, 5, 64, dtype=torch.float16)
    bias = torch.zeros(1, 3, 5, 7, dtype=torch.float16)
    view, copied = attn_mod._bias_view("bias", bias, (2, 3, 5, 7), q)  # noqa: SLF001
    assert view.stride() == (0, 35, 7, 1)
    assert view.data_ptr() == bias.data_ptr() and not copied
    view, copied = attn_mod._bias_view("bias", bias.transpose(2, 3).contiguous().transpose(2, 3), (2, 3, 5, 7), q)  # noqa: SLF001
    assert copied and view.stride(-1) == 1  # a last stride other than 1 is the one case that needs a copy
    with pytest.raises(ValueError, match="broadcast"):
        attn_mod._bias_view("bias", torch.zeros(4, 3, 5, 7, dtype=torch.float16), (2, 3, 5, 7), q)  # noqa: SLF001
    with pytest.raises(ValueError, match="float16"):
        attn_mod._bias_view("bias", torch.zeros(5, 7, dtype=torch.int32), (2, 3, 5, 7), q)  # noqa: SLF001


def test_tile_layout_pads_rows_only_where_needed() -> None:
    """The layout the kernel fetches in tiles: 16-bit, 16-byte aligned base, strides of the dimensions with more than
    one entry in multiples of 8. The reference builds its windowed blocks' bias that way itself (rows padded to a
    multiple of 8 and sliced, src/fastforks/_optimize/transformer.py:463-466)."""
    swin = torch.zeros(1, 12, 49, 56, dtype=torch.float16)[..., :49]  # the reference's `_swin_bias` layout
    assert ff.tile_layout(swin).data_ptr() == swin.data_ptr()  # taken as it is
    odd = torch.arange(2 * 3 * 5 * 7, dtype=torch.float32).reshape(2, 3, 5, 7).to(torch.bfloat16)
    padded = ff.tile_layout(odd)
    assert padded.shape == odd.shape and torch.equal(padded, odd)
    assert padded.stride() == (3 * 5 * 8, 5 * 8, 8, 1) and padded.data_ptr() % 16 == 0
    assert ff.tile_layout(padded).data_ptr() == padded.data_ptr()  # idempotent
    # fewer dims are taken as broadcast over batch and heads; the stride of a dimension of one entry does not matter
    two_d = ff.tile_layout(torch.zeros(5, 7, dtype=torch.float16))
    assert two_d.shape == (1, 1, 5, 7) and two_d.stride(2) == 8
    single_row = torch.zeros(1, 1, 1, 7, dtype=torch.float16)
    assert ff.tile_layout(single_row).data_ptr() == single_row.data_ptr()
    with pytest.raises(ValueError, match="float16 / bfloat16"):
        ff.tile_layout(torch.zeros(5, 7))
    # `attention` pads a 16-bit bias itself and reports the copy; a float32 bias is passed through for the row-wise loads
    q = torch.zeros(2, 3, 5, 64, dtype=torch.float16)
    view, copied = attn_mod._bias_view("bias", odd.half(), (2, 3, 5, 7), q, tiled=True)  # noqa: SLF001
    assert copied and view.stride(2) == 8
    view, copied = attn_mod._bias_view("bias", odd.float(), (2, 3, 5, 7), q, tiled=True)  # noqa: SLF001
    assert not copied and view.stride(2) == 7


def test_rope_table_and_contract_on_the_host() -> None:
    """`rope_table` is plain torch and runs anywhere; `rope_qk_` rejects what the kernel cannot take before any launch."""
    import numpy as np

    from oracle import rope_oracle as ro

    cs = ff.rope_table(3, 4, 100.0)
    assert cs.shape == (12, 2, 32) and cs.dtype == torch.float32
    np.testing.assert_allclose(cs.numpy(), ro.rope_table(3, 4, 100.0), rtol=0, atol=2e-6)
    with pytest.raises(ValueError, match="CUDA"):
        ff.rope_qk_(torch.zeros(1, 17, 3, 2, 64, dtype=torch.float16), cs)


def test_resolve_mode_follows_the_reference_rule(caplog: pytest.LogCaptureFixture) -> None:
    assert ff.resolve_mode("portable") == "portable"
    with pytest.raises(ValueError, match="mode"):
        ff.resolve_mode("fast")
    if not torch.cuda.is_available():
        with caplog.at_level("INFO", logger="fastforks_b200"):
            assert ff.resolve_mode("auto") == "portable"  # logged, never silent
        assert "using portable" in caplog.text
        with pytest.raises(ff.BackendUnavailableError, match="no CUDA device"):
            ff.resolve_mode("kernels")


def test_missing_library_fails_loudly(monkeypatch: pytest.MonkeyPatch, tmp_path) -> None:  # noqa: ANN001
    from fastforks_b200 import _lib

    monkeypatch.setattr(_lib, "SHARED_OBJECT", tmp_path / "absent.so")
    _lib.library.cache_clear()
    try:
        with pytest.raises(ff.KernelUnavailableError, match="not built"):
            _lib.library()
    finally:
        _lib.library.cache_clear()


def test_host_attention_contract_is_checked_before_any_copy() -> None:
    """`HostAttention.check` is host logic only: it needs no device and rejects what the copies could not take."""
    check = ff.HostAttention.check
    x = torch.zeros(2, 5, 3, 4, 64, dtype=torch.float16)
    o = torch.zeros(2, 5, 4, 64, dtype=torch.float16)
    check([], [])
    with pytest.raises(ValueError, match="outputs"):
        check([x], [])
    with pytest.raises(ValueError, match="packed"):
        check([x[:, :, 0]], [o])
    with pytest.raises(ValueError, match="expected"):
        check([x], [o[:, :4].contiguous()])
    with pytest.raises(ValueError, match="float16"):
        check([x.float()], [o.float()])
    with pytest.raises(ValueError, match="contiguous"):
        check([x.transpose(0, 1).contiguous().transpose(0, 1)], [o])
    with pytest.raises(ValueError, match="differs"):
        check([x, torch.zeros(1, 5, 3, 4, 64, dtype=torch.float16)], [o, torch.zeros(1, 5, 4, 64, dtype=torch.float16)])
    with pytest.raises(ValueError, match="empty"):
        check([x[:0]], [o[:0]])
