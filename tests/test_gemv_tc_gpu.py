"""The opt-in tensor-memory decode kernel (KQ_GEMV_TC=1) against the default decode kernel.

The lever is read once per process, so the opt-in run happens in a child process."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

_CHILD = r"""
import sys, numpy as np, torch
import mlx_kquant_b200 as kq
from mlx_kquant_b200.synth import random_wire
out = sys.argv[1]
res = {}
for (N, K, M) in ((128, 256, 1), (1000, 2048, 1), (4096, 4096, 2), (512, 14336, 1)):
    W = random_wire('q4_k', N, K, seed=11)
    x = torch.randn(M, K, device='cuda', generator=torch.Generator('cuda').manual_seed(5)).half()
    res[f'{N}_{K}_{M}'] = kq.quantized_matmul(x, W, None, 'q4_k').float().cpu().numpy()
np.savez(out, **res)
"""


def _run(tmp_path, name, env_extra):
    out = tmp_path / name
    env = dict(os.environ, **env_extra)
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__))), env.get("PYTHONPATH", "")])
    subprocess.run([sys.executable, "-c", _CHILD, str(out)], check=True, env=env, timeout=300)
    return np.load(str(out))


def test_tensor_memory_decode_matches_default(tmp_path):
    base = _run(tmp_path, "base.npz", {"KQ_GEMV_TC": "0"})
    tc = _run(tmp_path, "tc.npz", {"KQ_GEMV_TC": "1"})
    for k in base.files:
        a, b = base[k].astype(np.float64), tc[k].astype(np.float64)
        # both round an fp32 sum to fp16 once; the sums differ only in accumulation order
        assert np.linalg.norm(a - b) <= 1e-3 * np.linalg.norm(a), k
        assert np.abs(a - b).max() <= 2e-3 * np.abs(a).max(), k
