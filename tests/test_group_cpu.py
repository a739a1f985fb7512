"""Host logic of the device group that needs no GPU: the rule that cuts a minibatch over shards."""
import os
import shutil
import subprocess

import pytest

from primitiv_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_batch_partition_rule(tmp_path):
    """tests/cpp/partition_check.cc over primitiv_b200/device/batch_partition.h: ranges tile the batch,
    are balanced, owner() inverts range(), and an even cut is primitiv's batch::split."""
    exe = str(tmp_path / "partition_check")
    subprocess.run(["g++", "-std=c++11", "-O2", "-I", os.path.join(ROOT, "primitiv_b200", "device"),
                    os.path.join(ROOT, "tests", "cpp", "partition_check.cc"), "-o", exe], check=True, timeout=300)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.startswith("ok 9600"), r.stdout + r.stderr


def test_even_cut_matches_the_multi_process_sharding():
    """Where the shard count divides the batch, the in-process group and the one-process-per-GPU
    sharding (primitiv_b200/sharding.py) give a rank the same items."""
    for world in (1, 2, 4, 8):
        for per in (1, 3, 8):
            total = world * per
            if total == 1:
                continue
            for rank in range(world):
                first, count = sharding.shard_range(total, rank, world)
                assert (first, first + count) == (rank * total // world, (rank + 1) * total // world)
