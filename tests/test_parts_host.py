"""Host-side facts of the parts that need no GPU: the rotary part's table of frequencies."""
import math

import torch

from hymt2sharp_b200.parts.rope import NeoXRotary


def test_rotary_frequencies_and_their_sharing():
    """f_i = base^(-i / half) in float32 (src/HyMT2Sharp/Ops.cs:175-177); layers with equal frequencies share one
    tensor, so that what a step works out from it (the angles of its tokens) serves all of them."""
    a, b = NeoXRotary(128, 128, 10000.0), NeoXRotary(128, 128, 10000.0)
    c, d = NeoXRotary(128, 128, 5e6), NeoXRotary(128, 64, 10000.0)
    for part in (a, b, c, d):
        part.load({}, "cpu", torch.float32)
    epi = a.kernel_epilogue(None)
    table, rope_dim = epi.inv_freq, epi.rope_dim
    assert epi.pairing == "half"
    assert rope_dim == 128 and table.dtype == torch.float32 and table.shape == (64,)
    want = [1.0 / math.pow(10000.0, i / 64) for i in range(64)]
    assert torch.allclose(table.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6)
    assert b.kernel_epilogue(None).inv_freq.data_ptr() == table.data_ptr()
    assert c.kernel_epilogue(None).inv_freq.data_ptr() != table.data_ptr()
    assert d.kernel_epilogue(None).inv_freq.data_ptr() != table.data_ptr() and d.kernel_epilogue(None).inv_freq.shape == (32,)
