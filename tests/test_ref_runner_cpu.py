"""The executed-reference timing harness (oracle/ref_runner.py) must work from inside a launcher's worker:
the launcher's rendezvous variables must not leak into the CPU ranks it starts."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ditango", "core", "attention.py")),
                    reason="the copy of the reference's attention path has not been made (oracle/make_ref.py)")
def test_reference_arm_under_a_launcher_environment():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29999", WORLD_SIZE="2", RANK="0", LOCAL_RANK="0",
               TORCHELASTIC_USE_AGENT_STORE="True", TORCHELASTIC_RUN_ID="none", OMP_NUM_THREADS="1")
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from oracle import ref_runner as R\n"
            "r = R.time_reference(2, dict(B=1, S=256, H=2, D=64, dividers=[1, 2, 2, 1], bf16=False, seed=0), limit_s=120)\n"
            "assert r['steps'] == 4 and r['flops'] > 0 and r['seconds'] > 0, r\n"
            "import os; assert os.environ['MASTER_PORT'] == '29999' and os.environ['TORCHELASTIC_USE_AGENT_STORE'] == 'True'\n"
            "print('ok')\n" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ditango", "core", "attention.py")),
                    reason="the copy of the reference's attention path has not been made (oracle/make_ref.py)")
@pytest.mark.parametrize("world,seed", [(4, 0), (4, 1), (8, 2)])
def test_oracle_equals_the_executed_reference_on_random_legal_schedules(world, seed):
    """Beyond the committed fixtures: the reference's own proAttention.attn, run here on gloo ranks, against the
    oracle on fresh random schedules (legalised and screened) and inputs; fp32 on both sides."""
    import numpy as np
    import torch
    from oracle import ref_runner as R
    from oracle import ring_oracle as O
    from ditango_b200.core import redundancy_map as rmod
    from ditango_b200.core.config import init_config
    rng = np.random.RandomState(seed)
    T = 8
    legal = [d for d in (2, 4, 8) if d <= world]
    div = np.ones((T, 1), dtype=np.int64)
    for t in range(1, T):
        if rng.rand() < 0.7:
            div[t, 0] = legal[rng.randint(len(legal))]
    cfg = init_config(None, make_output_dir=False)
    cfg.num_layers, cfg.num_inference_steps = 1, T
    rmod.destroy_redundancy_map()
    rm = rmod.init_redundancy_map(cfg, world_size=world)
    rm.divider_map = torch.from_numpy(div)
    rm._refine_divider_map()
    rm.screen_self_sends()
    col = [int(x) for x in rm.get_map()[:, 0].tolist()]
    rmod.destroy_redundancy_map()
    B, S, H, D = 1, 16 * world, 2, 32
    data = O.drifting_qkv(B, S, H, D, T, seed=10 + seed, drift=0.05)
    got = R.time_reference(world, dict(B=B, S=S, H=H, D=D, dividers=col, bf16=False, data=data, collect=True), limit_s=240)
    want, _ = O.run_ring_group(world, col, data)
    for r in range(world):
        for t in range(T):
            err = np.abs(got["outputs"][r][t] - want[t][r].numpy()).max()
            assert err <= 2e-5, (col, r, t, err)


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ditango", "core", "attention.py")),
                    reason="the copy of the reference's attention path has not been made (oracle/make_ref.py)")
def test_oracle_equals_the_executed_reference_on_a_packed_batch():
    """The packed path (varlen_attn) live: four ranks, each with a valid and a pad segment of its own, dividers
    through a reuse phase; compared on the valid rows (a pad row that meets an empty key segment is undefined in
    the reference)."""
    import numpy as np
    from oracle import ref_runner as R
    from oracle import ring_oracle as O
    world, col = 4, [1, 1, 2, 2, 1, 4, 4, 1]
    B, S, H, D = 1, 24 * world, 2, 32
    lo = S // world
    cu = [[0, lo - 5, lo], [0, lo - 9, lo], [0, lo, lo], [0, lo - 3, lo]]
    data = O.drifting_qkv(B, S, H, D, len(col), seed=21, drift=0.05)
    got = R.time_reference(world, dict(B=B, S=S, H=H, D=D, dividers=col, bf16=False, data=data, collect=True, cu=cu),
                           limit_s=240)
    want, _ = O.run_ring_group(world, col, data, cu_per_rank=cu)
    for r in range(world):
        valid = cu[r][1]
        for t in range(len(col)):
            err = np.abs(got["outputs"][r][t][0, :valid] - want[t][r][:valid].numpy()).max()
            assert err <= 2e-5, (r, t, err)
