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
