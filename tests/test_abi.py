"""The C-ABI library: builds, loads, exports every symbol the header declares, and its host
logic (geometry, argument checks) behaves.  No compute calls: CPU only."""
import ctypes as C
import re
from pathlib import Path

import pytest

import backup_1_b200 as b
from backup_1_b200 import lib as blib
from oracle import oracle as o

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "decxb.h").read_text()
    return sorted(set(re.findall(r"DECXB_API\s+[\w\s\*]+?\b(decxb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = b.load_library()
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/decxb.h but not exported"
    assert set(names) == set(blib.SIGNATURES), "python prototypes out of sync with the header"


def test_status_strings_and_version():
    L = b.load_library()
    assert L.decxb_version().startswith(b"decxb")
    assert b"initialized" in L.decxb_status_string(1)
    assert b"dims" in L.decxb_status_string(3)


def test_no_device_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(b.DecxbError) as e:
        b.Context(0)
    assert e.value.status in (101, 102)


@pytest.mark.parametrize("W,H,depth,kW,kH,N,flag", [
    (224, 224, 64, 3, 3, 64, 1), (56, 56, 256, 3, 3, 256, 1), (22, 19, 6, 3, 5, 5, 0), (9, 7, 3, 3, 3, 2, 1),
])
def test_conv_geometry_matches_oracle(W, H, depth, kW, kH, N, flag):
    g = b.conv_geometry(W, H, depth, kW, kH, N, flag)
    ow, oh, eq, M, Kp = o.conv_geometry(W, H, depth, kW, kH, flag)
    assert (g.out_w, g.out_h, g.eq_w, g.M, g.Kp, g.Np) == (ow, oh, eq, M, Kp, o.ceil4(N))


def test_conv_geometry_rejects_bad_input():
    for args, status in [((8, 8, 4, 19, 3, 1, 1), 5), ((8, 8, 4, 3, 3, 1, 7), 11), ((2, 2, 4, 3, 3, 1, 0), 5), ((0, 8, 4, 3, 3, 1, 1), 13)]:
        with pytest.raises(b.DecxbError) as e:
            b.conv_geometry(*args)
        assert e.value.status == status


def test_config_sizes_of_baseline():
    g3 = b.conv_geometry(224, 224, 64, 3, 3, 64, 1)
    assert (g3.M, g3.Kp) == (50176, 576) and g3.M * g3.Kp * 4 == 115605504
    g4 = b.conv_geometry(56, 56, 256, 3, 3, 256, 1)
    assert (g4.M, g4.Kp) == (3136, 2304) and g4.M * g4.Kp * 4 == 28901376
