"""One elementwise operator through the runtime, as the reference's quickstart does
(examples/tutorial/quickstart_tutorial.py)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import ark_b200 as ark  # noqa: E402


def main():
    ark.init()
    m, n = 64, 64
    a = ark.tensor([m, n], ark.fp16)
    b = ark.tensor([m, n], ark.fp16)
    c = ark.add(a, b)
    runtime = ark.Runtime()
    runtime.launch()
    ha, hb = np.random.rand(m, n).astype(np.float16), np.random.rand(m, n).astype(np.float16)
    a.from_numpy(ha)
    b.from_numpy(hb)
    runtime.run()
    np.testing.assert_allclose(c.to_numpy(), ha + hb)
    runtime.stop()
    runtime.reset()
    print("quickstart ok")


if __name__ == "__main__":
    main()
