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


# ---- split plan of the CUDA-core weight gradient: sizing and launch share one source of truth -----

RESNET32_LAYERS = [  # (M = batch 256 x output positions, K = C_in * 9, N = C_out, T at max_input_size 256)
    (262144, 27, 16, 1), (262144, 144, 16, 1),
    (65536, 144, 32, 1), (65536, 288, 32, 2), (65536, 16, 32, 1),
    (16384, 288, 64, 2), (16384, 576, 64, 3), (16384, 32, 64, 1),
    (256, 64, 10, 1),
]


def _plan(lib, m, k, n, t):
    import ctypes
    splits, rows = ctypes.c_int32(), ctypes.c_int32()
    assert lib.al_wgrad_split_plan(m, k, n, t, ctypes.byref(splits), ctypes.byref(rows)) == 0
    return splits.value, rows.value


def test_wgrad_split_plan_fits_the_scratch_it_is_sized_with():
    """The partial sums of a split weight gradient must fit what ``al_backward_scratch_floats``
    promises for the same layer, whatever tile table the launch itself runs with (a call without
    a clamp mask runs one GEMM over the whole K range: the plan may not depend on that)."""
    import os
    import random

    import pytest

    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built")
    lib = _lib.load()
    rng = random.Random(0)
    shapes = list(RESNET32_LAYERS)
    for _ in range(400):
        k = rng.choice([3, 27, 64, 144, 288, 576, 1000, 1024, 4096])
        shapes.append((rng.choice([1, 17, 512, 2048, 16384, 65536, 262144, 300001]), k,
                       rng.choice([1, 10, 16, 32, 33, 64, 100, 1024]), rng.choice([1, 2, 3, 7, min(k, 16)])))
    for m, k, n, t in shapes:
        splits, rows = _plan(lib, m, k, n, t)
        assert splits >= 1 and rows % 16 == 0
        assert splits * rows >= m                      # the splits cover every row
        assert splits == 1 or (splits - 1) * rows < m  # and none of them starts beyond the last
        fixed = lib.al_backward_scratch_floats(m, k, n, t) - (splits * n * k if splits > 1 else 0)
        # the fixed part (bias / range / clip reductions) does not depend on K
        assert fixed == lib.al_backward_scratch_floats(m, 1, n, t) - (
            _plan(lib, m, 1, n, t)[0] * n if _plan(lib, m, 1, n, t)[0] > 1 else 0)
        assert fixed > 0


def test_backward_refuses_a_scratch_buffer_that_is_too_small():
    """Capacity travels with the pointer: a call whose scratch holds fewer floats than
    ``al_backward_scratch_floats`` asks for is refused on the host, before any launch."""
    import ctypes
    import os

    import pytest

    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built")
    lib = _lib.load()
    m, k, n, t = 65536, 288, 32, 2
    desc = _lib.AlDesc()
    desc.M, desc.K, desc.N, desc.T = m, k, n, t
    desc.dtype = _lib.AL_F32
    desc.inp_res, desc.out_res, desc.out_bound = -1.0, -1.0, -1.0
    args = _lib.AlBackwardArgs()
    args.tile_ends = (ctypes.c_int32 * 2)(144, 288)
    args.grad_out = 256  # never dereferenced: the call must fail before any launch
    args.reduce_scratch = 256
    args.reduce_scratch_floats = lib.al_backward_scratch_floats(m, k, n, t) - 1
    assert lib.al_backward(desc, args, None) == _lib.AL_ERR_BAD_ARGUMENT
    assert b"reduce_scratch holds" in lib.al_last_error()


def test_direct_convolution_input_gradient_says_which_layers_it_covers():
    """``al_conv2d_input_grad_supported`` is host arithmetic (geometry, divisibility, shared-memory budget): the
    unit-stride fp32 convolutions of ResNet-32 qualify, strided / dilated / bf16 layers and ragged channel counts
    take the patch-gradient route."""
    lib = _lib.load()
    ok = lib.al_conv2d_input_grad_supported
    for cin, cout, size in ((16, 16, 32), (32, 32, 16), (64, 64, 8), (16, 32, 32)):
        assert ok(_lib.AL_F32, cout, 256, cin, size, size, 3, 3, 1, 1, 1, 1, 1, 1) == 1
    assert ok(_lib.AL_BF16, 16, 256, 16, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1) == 0
    assert ok(_lib.AL_F32, 32, 256, 16, 32, 32, 3, 3, 2, 2, 1, 1, 1, 1) == 0      # strided
    assert ok(_lib.AL_F32, 16, 256, 16, 32, 32, 3, 3, 1, 1, 2, 2, 2, 2) == 0      # dilated
    assert ok(_lib.AL_F32, 16, 256, 16, 32, 32, 3, 3, 1, 1, 3, 3, 1, 1) == 0      # padding as large as the kernel
    assert ok(_lib.AL_F32, 10, 256, 16, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1) == 0      # output channels not a multiple of 4
    assert ok(_lib.AL_F32, 16, 256, 3, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1) == 0       # three input channels
    assert ok(_lib.AL_F32, 16, 0, 16, 32, 32, 3, 3, 1, 1, 1, 1, 1, 1) == 0        # no image
    # wide layers: the weights of a channel chunk must fit 96 KB of shared memory next to the staged rows
    assert ok(_lib.AL_F32, 256, 8, 256, 14, 14, 3, 3, 1, 1, 1, 1, 1, 1) == 0


def test_pair_kernel_work_list_covers_every_block_once():
    """The backward GEMMs on CTA pairs walk a list of whole blocks followed, when the last round would be short, by
    the halves of its blocks: every block appears once as a whole or once per half, no pair gets more than one half
    block, and the list is only cut when it shortens the last round."""
    import ctypes

    lib = _lib.load()
    total, block, half = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()

    def items(num_blocks, n_pairs):
        assert lib.al_pair_work_item(num_blocks, n_pairs, 0, total, block, half) == _lib.AL_OK
        out = []
        for v in range(total.value):
            assert lib.al_pair_work_item(num_blocks, n_pairs, v, total, block, half) == _lib.AL_OK
            out.append((block.value, half.value))
        assert lib.al_pair_work_item(num_blocks, n_pairs, total.value, total, block, half) == _lib.AL_OK
        assert block.value == -1
        return out

    cut = 0
    for n_pairs in (1, 2, 7, 66, 70, 74):
        for num_blocks in list(range(1, 4 * n_pairs + 3)) + [256, 384, 432, 512, 768, 1024, 1152]:
            work = items(num_blocks, n_pairs)
            whole = [b for b, h in work if h < 0]
            halves = [(b, h) for b, h in work if h >= 0]
            assert whole == list(range(len(whole)))
            assert sorted(halves) == [(b, h) for b in range(len(whole), num_blocks) for h in (0, 1)]
            if halves:
                cut += 1
                rem = num_blocks % n_pairs
                assert len(whole) % n_pairs == 0 and len(whole) // n_pairs <= 3
                assert 0 < rem and 2 * rem <= n_pairs and len(halves) == 2 * rem
                # items of one pair: v = p, p + n_pairs, ...; the half blocks sit in the last round, one per pair
                assert all(v >= len(whole) for v, (b, h) in enumerate(work) if h >= 0)
            else:
                assert len(work) == num_blocks
    assert cut > 0
    # config 2's weight gradient: 256 blocks on 74 pairs -> 222 whole blocks and the last 34 as 68 halves
    work = items(256, 74)
    assert len(work) == 222 + 68 and work[221] == (221, -1) and work[222] == (222, 0) and work[-1] == (255, 1)
    assert lib.al_pair_work_item(0, 74, 0, total, block, half) == _lib.AL_ERR_BAD_ARGUMENT
