"""The host side of the kernels' failure reporting: a status pair read back beside a step's
tokens becomes an exception that names the kernel family, the code and the block."""
import pytest

from kvcm.kernels import library as K


def test_healthy_status_raises_nothing():
    K.raise_on_status(0, 0)


def test_status_pair_names_family_code_and_block(monkeypatch):
    cleared = []
    monkeypatch.setattr(K, "clear_errors", lambda: cleared.append(True))
    with pytest.raises(K.KernelError, match=r"gemm_stream: a bounded wait ran out .*code 2, block 37"):
        K.raise_on_status(1, (2 << 16) | 37)
    assert cleared == [True]                       # the words are cleared before the exception leaves
    with pytest.raises(K.KernelError, match=r"attention_tcgen05: .*code 7, block 3"):
        K.raise_on_status(5, (7 << 16) | 3)
    assert "family 9" in K.describe_status(9, 1 << 16)
    assert len(K.STATUS_FAMILIES) == 5
