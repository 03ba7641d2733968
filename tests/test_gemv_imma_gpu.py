"""The integer tensor-pipe q4_k decode kernel (lever KQ_GEMV_IMMA) against the fp64 product of the
dequantized weights, and against the run with the lever off.

The lever is read once per process, so each setting runs in a child process."""
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
cases = [(128, 256, 1, 'f16'), (1000, 2048, 1, 'f16'), (4096, 4096, 2, 'f16'), (515, 14336, 1, 'bf16'),
         (4100, 4096, 1, 'f32'), (9600, 1024, 1, 'f16'), (33, 16384, 2, 'bf16'), (20000, 512, 2, 'f16')]
DT = {'f16': torch.float16, 'bf16': torch.bfloat16, 'f32': torch.float32}
for (N, K, M, dt) in cases:
    W = random_wire('q4_k', N, K, seed=11)
    x = (torch.randn(M, K, device='cuda', generator=torch.Generator('cuda').manual_seed(5)) * 2.5).to(DT[dt])
    if (N, dt) == (1000, 'f16'):
        x[0, 300:333] = 0          # a whole sub-block of zeros and an outlier
        x[0, 7] = 900.0
    y = kq.quantized_matmul(x, W, None, 'q4_k')
    xr = x.to(torch.bfloat16).double() if dt == 'f32' else x.double()
    ref = xr @ kq.dequantize(W, None, 'q4_k', dtype=torch.float32).double().T
    res[f'y_{N}_{K}_{M}_{dt}'] = y.float().cpu().numpy()
    res[f'r_{N}_{K}_{M}_{dt}'] = ref.cpu().numpy()
# non-finite activations propagate
W = random_wire('q4_k', 64, 512, seed=12)
x = torch.ones(1, 512, device='cuda', dtype=torch.float16)
x[0, 100] = float('inf')
res['inf'] = kq.quantized_matmul(x, W, None, 'q4_k').float().cpu().numpy()
np.savez(out, **res)
"""


def _run(tmp_path, name, env_extra):
    out = tmp_path / name
    env = dict(os.environ, **env_extra)
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__))), env.get("PYTHONPATH", "")])
    subprocess.run([sys.executable, "-c", _CHILD, str(out)], check=True, env=env, timeout=300)
    return np.load(str(out))


def test_integer_tensor_pipe_decode(tmp_path):
    on = _run(tmp_path, "on.npz", {"KQ_GEMV_IMMA": "1"})
    off = _run(tmp_path, "off.npz", {"KQ_GEMV_IMMA": "0"})
    for k in on.files:
        if not k.startswith("y_"):
            continue
        y, ref = on[k].astype(np.float64), on["r" + k[1:]].astype(np.float64)
        tol = 2e-3 if k.endswith("_f16") else 4e-3   # bf16 outputs carry a 2^-9 rounding of their own
        assert np.linalg.norm(y - ref) <= tol * np.linalg.norm(ref), k
        b = off[k].astype(np.float64)
        assert np.linalg.norm(y - b) <= tol * np.linalg.norm(b), k
    assert not np.isfinite(on["inf"]).any()
