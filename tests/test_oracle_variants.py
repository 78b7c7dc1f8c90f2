"""Oracle restatements of the complex / positive-real loop references against the reference's own outputs."""
import numpy as np
import torch

from oracle import variants as V
from tests.helpers import load_golden


def test_loop_restatements_match_reference_outputs():
    g = load_golden("loop_variants")
    u, dt, z, D = g["u"], g["dt"], g["z"], g["D"]
    y = V.preal_ref(u, dt, g["x_rho"], g["B_real"], g["C_real"], D, z)
    torch.testing.assert_close(y, g["y_preal"], rtol=2e-5, atol=2e-5)
    x = torch.stack([g["x_rho"], g["x_theta"]])
    y = V.complex_ref(u, dt, x, g["B_complex"], g["C_complex"], D, z)
    torch.testing.assert_close(y, g["y_complex"], rtol=2e-5, atol=2e-5)
