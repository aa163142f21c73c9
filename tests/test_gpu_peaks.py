"""Measured issue-rate ceilings of the device (`-m gpu`)."""
import pytest
import torch

from raygaussx_b200 import _lib

pytestmark = pytest.mark.gpu


def test_measured_issue_peaks_are_plausible():
    """FMA and ex2 rates of the register-chain kernels: within the range a current data-centre GPU can have
    (the derived B200 figures are 74 TFLOP/s and 4,650 G ex2/s)."""
    import ctypes as C
    fma, ex2 = C.c_float(), C.c_float()
    assert _lib.lib().rgx_measure_peaks(torch.cuda.current_device(), C.byref(fma), C.byref(ex2)) == 0
    assert 20.0 < fma.value < 120.0, fma.value
    assert 1000.0 < ex2.value < 8000.0, ex2.value
