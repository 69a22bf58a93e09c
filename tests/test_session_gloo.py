"""The wire message across a real process boundary (two gloo ranks on CPU): page-granular pieces of a session delivered
out of order and in two batches, the decode side handing pages over as their pieces arrive, a damaged piece refused by
its checksum and sent again (engine/src/session.rs:194-200 is the message's field set; "page-granular and resumable,
partial transfer visible as a partially filled block table" is the reference's plan for it)."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_pieces_cross_a_process_boundary_out_of_order_and_resume(tmp_path):
    out = tmp_path / "result.txt"
    env = dict(os.environ, GLOO_RESULT=str(out), OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "gloo_session_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert out.read_text().startswith("OK wire")
