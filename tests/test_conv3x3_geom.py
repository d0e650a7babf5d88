"""Implicit-GEMM tiling of 3x3 convolutions (csrc/gc_conv_geom.h): emulate the TMA boxes on the CPU and compare the
tile-by-tile GEMM with torch's convolution."""
import ctypes

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from gradient_compression_b200.ops import _native as nat


def _geom(n, h, w, c):
    out = (ctypes.c_int * 6)()
    ok = nat.host().gc_host_conv3x3_geom(n, h, w, c, out)
    return (dict(zip(("box_w", "box_h", "box_n", "cblocks", "tiles", "kblocks"), out)) if ok else None)


def _box(x_nhwc, coord, g):
    """What a 4-D TMA box load returns: out-of-range positions read as zero."""
    n_, h_, w_, c_ = x_nhwc.shape
    c0, w0, h0, n0 = coord
    box = np.zeros((g["box_n"], g["box_h"], g["box_w"], 32), dtype=np.float64)
    for dn in range(g["box_n"]):
        for dh in range(g["box_h"]):
            for dw in range(g["box_w"]):
                n, h, w = n0 + dn, h0 + dh, w0 + dw
                if 0 <= n < n_ and 0 <= h < h_ and 0 <= w < w_:
                    box[dn, dh, dw] = x_nhwc[n, h, w, c0:c0 + 32]
    return box.reshape(128, 32)            # rows in (n, h, w) order = the tile's output positions


@pytest.mark.parametrize("n,h,w,cin,cout", [(2, 32, 32, 32, 8), (3, 16, 16, 64, 16), (5, 8, 8, 32, 8), (20, 4, 4, 32, 8),
                                            (1, 64, 64, 32, 4), (3, 2, 64, 32, 4)])
def test_tilewise_gemm_equals_convolution(n, h, w, cin, cout):
    g = _geom(n, h, w, cin)
    assert g is not None and g["box_w"] * g["box_h"] * g["box_n"] == 128
    gen = torch.Generator().manual_seed(n * h + w + cin)
    x = torch.randn(n, cin, h, w, generator=gen, dtype=torch.float64)
    wt = torch.randn(cout, cin, 3, 3, generator=gen, dtype=torch.float64)
    ref = F.conv2d(x, wt, padding=1).permute(0, 2, 3, 1).reshape(n * h * w, cout).numpy()
    x_nhwc = x.permute(0, 2, 3, 1).contiguous().numpy()
    b = wt.permute(0, 2, 3, 1).reshape(cout, 9 * cin).numpy()          # channels-last filter read as [Cout, 9 * Cin]
    out = np.zeros((g["tiles"] * 128, cout))
    coord = (ctypes.c_int * 4)()
    for tile in range(g["tiles"]):
        acc = np.zeros((128, cout))
        for kb in range(g["kblocks"]):
            assert nat.host().gc_host_conv3x3_box(n, h, w, cin, tile, kb, coord)
            assert coord[0] % 4 == 0                                    # innermost TMA coordinate: 16-byte aligned
            acc += _box(x_nhwc, list(coord), g) @ b[:, kb * 32:(kb + 1) * 32].T
        out[tile * 128:(tile + 1) * 128] = acc
    assert np.allclose(out[:n * h * w], ref, atol=1e-9)


def test_shapes_outside_the_tiling_are_refused():
    assert _geom(4, 7, 7, 32) is None           # width does not divide 128
    assert _geom(4, 3, 32, 32) is None          # an image is neither whole tiles nor a divisor of a tile
    assert _geom(4, 8, 8, 48) is None           # channels not a multiple of 32
    assert _geom(4, 8, 8, 64) is not None
