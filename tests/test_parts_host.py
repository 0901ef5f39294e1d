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
    table, rope_dim = a.rotary_table()
    assert rope_dim == 128 and table.dtype == torch.float32 and table.shape == (64,)
    want = [1.0 / math.pow(10000.0, i / 64) for i in range(64)]
    assert torch.allclose(table.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6)
    assert b.rotary_table()[0].data_ptr() == table.data_ptr()
    assert c.rotary_table()[0].data_ptr() != table.data_ptr()
    assert d.rotary_table()[0].data_ptr() != table.data_ptr() and d.rotary_table()[0].shape == (32,)
