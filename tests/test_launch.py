"""Job launcher: environment of the workers, failure propagation, ssh command construction."""
import os
import subprocess
import sys

import pytest

from mxnet_b200.parallel import launch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.integration
def test_local_launch_runs_gloo_ranks(tmp_path):
    script = tmp_path / 'w.py'
    script.write_text(
        "import os, sys\n"
        "sys.path.insert(0, %r)\n"
        "from mxnet_b200.parallel import dist\n"
        "import torch\n"
        "dist.ensure_initialized('gloo')\n"
        "t = torch.ones(1) * (dist.rank() + 1)\n"
        "dist.all_reduce_sum(t)\n"
        "assert os.environ['DMLC_ROLE'] == 'worker' and os.environ['DMLC_NUM_WORKER'] == '3'\n"
        "open(os.path.join(%r, 'out%%d' %% dist.rank()), 'w').write(str(float(t)))\n"
        "dist.destroy()\n" % (os.path.dirname(HERE), str(tmp_path)))
    rc = launch.main(['-n', '3', '--env', 'CUDA_VISIBLE_DEVICES=', sys.executable, str(script)])
    assert rc == 0
    assert [open(str(tmp_path / ('out%d' % r))).read() for r in range(3)] == ['6.0'] * 3


def test_failure_of_one_worker_is_reported(tmp_path):
    script = tmp_path / 'f.py'
    script.write_text("import os, sys, time\nif os.environ['RANK'] == '1':\n    sys.exit(7)\ntime.sleep(30)\n")
    rc = launch.main(['-n', '2', sys.executable, str(script)])
    assert rc == 7


def test_ssh_command_lines():
    cmds = launch.ssh_commands(4, ['hostA', 'hostB'], ['python', 'train.py', '--x', 'a b'], 9000)
    assert len(cmds) == 4 and cmds[0][:4] == ['ssh', '-o', 'StrictHostKeyChecking=no', 'hostA'] and cmds[2][3] == 'hostB'
    assert 'RANK=2' in cmds[2][4] and 'LOCAL_RANK=0' in cmds[2][4] and 'MASTER_ADDR=hostA' in cmds[2][4]
    assert "'a b'" in cmds[3][4] and 'WORLD_SIZE=4' in cmds[3][4]
