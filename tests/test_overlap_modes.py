"""The backward pass may overlap its row-moving tail with the weight-gradient GEMMs
(MOE_B200_OVERLAP = 0, 1, 2); every mode must give the same results as the plain order."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode", ["0", "1", "2"])
def test_every_overlap_mode_matches_the_checker(mode):
    env = dict(os.environ, MOE_B200_OVERLAP=mode)
    r = subprocess.run([sys.executable, os.path.join(HERE, "overlap_child.py")], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "overlap mode %s ok" % mode in r.stdout
