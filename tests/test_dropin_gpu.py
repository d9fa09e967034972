"""Drop-in check on the GPU: the reference's own three drivers (its test/*.cu compiled unchanged against
include/ and linked to libet_b200.so; built into oracle/_ref/ where the reference checkout is available) run to
completion, and this repository's example drivers run and report finite outputs."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", ["tile", "prune", "length"])
def test_reference_drivers_run_against_this_library(name):
    exe = os.path.join(ROOT, "oracle", "_ref", f"dropin_encoder_{name}_test")
    if not os.path.exists(exe):
        pytest.skip("drop-in drivers not built (no reference checkout at build time)")
    # seq_len >= d_model: the reference's drivers size their LayerNorm vectors by seq_len (test/tile_test.cu:29-30)
    res = subprocess.run([exe, "1024", "16", "1024", "0.8"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr


@pytest.mark.parametrize("name,args", [("encoder_tile_test", ["128", "12", "768", "0.75", "16", "5"]),
                                       ("encoder_prune_test", ["256", "12", "768", "0.5", "4", "5"]),
                                       ("encoder_prune_test", ["256", "12", "768", "0.5", "4", "5", "v"]),
                                       ("encoder_length_test", ["512", "12", "768", "0.75", "8", "3"])])
def test_example_drivers(name, args):
    exe = os.path.join(ROOT, "et_b200", "examples", "bin", name)
    if not os.path.exists(exe):
        pytest.skip("example drivers not built")
    res = subprocess.run([exe] + args, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "non-finite 0" in res.stdout
