"""Host-side plumbing of the operator that needs no GPU: descriptor and tile-table caching."""
import torch

from aihwkit_lightning_b200 import _lib
from aihwkit_lightning_b200.nn import functional as F
from aihwkit_lightning_b200.simulator.configs import TorchInferenceRPUConfig


def test_descriptors_are_cached_by_value_and_handed_out_as_copies():
    rpu = TorchInferenceRPUConfig()
    rpu.forward.inp_res = 254
    a = F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True)
    b = F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True)
    assert a is not b and bytes(a) == bytes(b)
    a.save_for_backward = 1                       # per-call fields do not leak into the cache
    assert F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True).save_for_backward == 0
    rpu.forward.inp_res = 14                      # the configuration object is mutable: its values are the key
    c = F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True)
    assert c.inp_res == 14 and b.inp_res == 254
    rpu.pre_post.input_range.enable = True
    rpu.pre_post.input_range.dynamic = True
    assert F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True).ir_mode == _lib.AL_IR_DYNAMIC
    with F.operator_settings(engine="simt", no_rounding=True):
        d = F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True)
        assert d.engine == _lib.AL_ENGINE_SIMT and d.no_rounding == 1
    e = F.make_desc(rpu, 4, 64, 32, 2, torch.float32, True)
    assert e.engine == _lib.AL_ENGINE_AUTO and e.no_rounding == 0
    assert F.make_desc(rpu, 4, 64, 32, 2, torch.bfloat16, False).dtype == _lib.AL_BF16


def test_tile_ends_are_cumulative_and_shared_per_tiling():
    a = _lib.tile_ends_array([3, 3, 2])
    assert list(a) == [3, 6, 8]
    assert _lib.tile_ends_array((3, 3, 2)) is a
    assert list(_lib.tile_ends_array([5])) == [5]
