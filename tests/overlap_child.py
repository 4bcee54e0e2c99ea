"""Child process of test_overlap_modes: two consecutive forward/backward passes with different
inputs under the overlap mode given by MOE_B200_OVERLAP, checked against the CPU checker.
Runs as a script so that the environment variable is read by a fresh copy of the library."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
from gpu_common import assert_routing_equal, make_pair, to_dev, to_np  # noqa: E402
from helpers import rel_l2  # noqa: E402
from oracle import GATE, DOWN, ROUTER, UP  # noqa: E402


def main():
    T, d, E, k, F = 300, 128, 8, 2, 96
    dev, ora, _ = make_pair(d, E, k, F, shared=True, precision="bf16", max_tokens=T, seed=5)
    g = np.random.Generator(np.random.Philox(21))
    worst = 0.0
    for step in range(3):      # the deferred weight gradients of pass i run beside the dispatch of pass i + 1
        x = torch.from_numpy(g.standard_normal((T, d)).astype(np.float32)).bfloat16().float().numpy()
        gy = torch.from_numpy(g.standard_normal((T, d)).astype(np.float32)).bfloat16().float().numpy()
        y, cache = dev.forward_train(to_dev(x, "bf16"))
        yo = ora.forward(x, logits=dev.router_cache(T)[0])   # same logits -> same routing decisions
        assert_routing_equal(cache, ora)
        dev.zero_grad()
        ora.zero_grad()
        gx = dev.backward(cache, to_dev(gy, "bf16"))
        gxo = ora.backward(gy)
        errs = [rel_l2(to_np(y), yo), rel_l2(to_np(gx), gxo)]
        for which, e in ((ROUTER, 0), (GATE, 1), (UP, 3), (DOWN, 6)):
            errs.append(rel_l2(dev.get_grad(which, e), ora.get_grad(which, e)))
        worst = max(worst, max(errs))
        assert max(errs) <= 2e-2, (step, errs)      # bf16 tolerance of the path
    dev.step_adam(lr=1e-3, step=1)                  # joins whatever is still on the side stream
    dev.synchronize()
    print("overlap mode %s ok, worst rel-L2 %.2e" % (os.environ.get("MOE_B200_OVERLAP", "default"), worst))


if __name__ == "__main__":
    main()
