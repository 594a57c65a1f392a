"""Opt-in transport variants on one GPU; collected last so that the established suites run first.

World 1 exercises the whole mechanism of the scattering GEMM epilogue on a single device: the
push writes the row map, the second expert GEMM (and the last dgrad GEMM) store every output row
through a per-row destination into the return slots, and the combine reduces from those slots.
The destinations are this GPU's own memory here; with more GPUs only the base addresses change
(``tests/test_gpu_fused_ep.py::test_epilogue_push_world2_equals_two_hop_pull``, opt-in).
"""
import pytest
import torch

from test_gpu_fused_ep import _close, _run

pytestmark = pytest.mark.gpu


def test_epilogue_push_world1_equals_local_kernels(native_ops, monkeypatch):
    """Bit-equal to the local kernels: same GEMM tiles, same reduction order, different route."""
    monkeypatch.setenv("TERRACE_EP_EPILOGUE_PUSH", "1")
    (rank, res, echo, x0, status, live), = _run(1, 1, 29781)
    assert status == 0
    assert live["epilogue_push_fwd"] == 1 and live["epilogue_push_bwd"] == 1
    for i, (a, b) in enumerate(zip(res["one_hop"], res["ref"])):
        if i == 2:      # gate gradients: same dot products, different lane partition
            _close(a, b, 1e-2)
        else:
            assert torch.equal(a, b)
    _close(echo, x0, 2e-2)
