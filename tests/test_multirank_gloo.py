"""World-size 2 and 4 on CPU (gloo): the pairing, the head / layer shares and the transfer
buffer layout used by the multi-GPU handoff, checked against one unsharded oracle run."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,case", [(2, "heads"), (4, "heads"), (4, "layers"), (2, "prefix")])
def test_ranks_tile_the_batch_and_match_the_oracle(tmp_path, world, case):
    out = tmp_path / "result.txt"
    env = dict(os.environ, GLOO_CASE=case, GLOO_RESULT=str(out), OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "gloo_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert out.read_text().startswith(f"OK {world} {case}")


def test_roles_cover_every_rank_once():
    from tempura_b200 import disagg
    for world in (1, 2, 4, 8):
        roles = [disagg.role_of(r, world, 80, 8) for r in range(world)]
        if world == 1:
            assert roles[0].is_prefill and roles[0].partner == 0 and roles[0].n_heads == 8
            continue
        P = world // 2
        assert [r.is_prefill for r in roles] == [True] * P + [False] * P
        for r in roles:
            assert roles[r.partner].partner == r.rank and roles[r.partner].pair == r.pair
            assert r.n_heads == 8 // P and r.head_begin == r.pair * (8 // P) and r.n_layers == 80
    with pytest.raises(Exception):
        disagg.role_of(0, 3, 80, 8)


def test_ranks_take_every_gpu_once_and_prefill_gpus_are_not_neighbours():
    """Slots of the pairing are placed on CUDA ordinals so that the GPUs reading host buffers (the prefill ranks) sit on
    every other ordinal, each next to its own decode rank; two ranks and the paired order keep rank r on GPU r."""
    from tempura_b200 import disagg
    for world in (1, 2, 4, 8):
        gpus = [disagg.gpu_of_rank(r, world) for r in range(world)]
        assert sorted(gpus) == list(range(world))
        assert [disagg.gpu_of_rank(r, world, "paired") for r in range(world)] == list(range(world))
        if world <= 2:
            assert gpus == list(range(world))
            continue
        for r in range(world):
            role = disagg.role_of(r, world, 80, 8)
            if role.is_prefill:
                assert gpus[r] == 2 * role.pair and gpus[role.partner] == gpus[r] + 1
    with pytest.raises(ValueError):
        disagg.gpu_of_rank(4, 4)
    with pytest.raises(ValueError):
        disagg.gpu_of_rank(0, 4, "striped")
