"""The C++ mirror of the reference's operator interface (OpDef -> CreateOp -> OpImpl::Compute),
exercised by a C++ test executable in the style of the reference's own *_test.cc programs
(tests/cpp/graph_ops_test.cc).  The executable is built by __graft_entry__.build()."""
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).parent / "cpp" / "bin"
EXE = BIN / "graph_ops_test"
FRONTEND = BIN / "frontend_test"


def _build(exe=EXE):
    if not exe.exists():
        import __graft_entry__ as g
        g.build()
    return exe


def test_registry_decls_and_scheduler_facade_cpu():
    r = subprocess.run([str(_build()), "cpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


@pytest.mark.gpu
def test_graph_ops_bit_exact_on_device(cuda):
    r = subprocess.run([str(_build()), "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


def test_vertex_function_recording_cpu():
    r = subprocess.run([str(_build(FRONTEND)), "cpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


@pytest.mark.gpu
def test_session_run_matches_oracle_on_device(cuda):
    """Tree-LSTM and chain LSTM declared through Sym / GraphSupport::Node(), one Session::Run training step each."""
    r = subprocess.run([str(_build(FRONTEND)), "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


VERTEX_OPS = BIN / "vertex_ops_test"


def test_standalone_vertex_ops_registered_and_compile_cpu():
    """MatMul / Add / Sub / Mul / Sigmoid / Tanh / Relu / Slice / Concat / Mirror under the reference's keys; the
    generated elementwise kernels compile for sm_100a without a GPU."""
    r = subprocess.run([str(_build(VERTEX_OPS)), "cpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout


@pytest.mark.gpu
def test_standalone_vertex_ops_on_device(cuda):
    r = subprocess.run([str(_build(VERTEX_OPS)), "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ok" in r.stdout
