"""GPU: training forward + backward (`diff_rasterize`) against the golden gradients produced by the reference
extension, against the live reference when it is built beside the repo, and basic autograd plumbing."""
import os

import numpy as np
import pytest

import harness
from htgs_b200 import scenes
from golden.make_golden import CASES, target_image

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GRAD_NAMES = ("positions", "scales", "rotations", "opacities", "sh_0", "sh_rest")
GRAD_RTOL = 1e-3    # gradients: relative to the largest magnitude of the tensor


def run_training_step(mod, scene, view, mode, K, densification_rows=0, use_distance_scaling=False):
    import torch
    tensors = harness.scene_tensors(scene)
    leaves = [t.clone().requires_grad_(True) for t in tensors]
    st = harness.settings_for(mod, scene, view, mode, K)
    dens = torch.zeros((densification_rows, scene.n, 1), device="cuda") if densification_rows else torch.empty(0, device="cuda")
    image = mod.diff_rasterize(*leaves, dens, st, use_distance_scaling)
    target = torch.from_numpy(target_image(view.height, view.width, 1000 + mode)).cuda()
    loss = (image - target).abs().mean()
    loss.backward()
    torch.cuda.synchronize()
    return image.detach(), [l.grad for l in leaves], dens


def assert_grads_close(ours, ref, what):
    for name, a, b in zip(GRAD_NAMES, ours, ref):
        a = a.detach().cpu().numpy() if hasattr(a, "detach") else np.asarray(a)
        b = b.detach().cpu().numpy() if hasattr(b, "detach") else np.asarray(b)
        assert a.shape == b.shape, f"{what} grad_{name}: shape {a.shape} vs {b.shape}"
        if b.size == 0:
            continue
        scale = np.abs(b).max()
        if scale == 0:
            assert np.abs(a).max() == 0, f"{what} grad_{name}: reference is all zero"
            continue
        err = np.abs(a - b).max() / scale
        assert err <= GRAD_RTOL, f"{what} grad_{name}: max error {err:.2e} of the tensor's scale"


def golden_cases():
    for name, case in CASES.items():
        for mode, K in case["modes"]:
            yield name, mode, K


@pytest.mark.parametrize("name,mode,K", list(golden_cases()))
def test_training_against_reference_golden(name, mode, K):
    scene = scenes.tiny_scene(**CASES[name]["kwargs"])
    view = scene.views[0]
    gold = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    tag = f"m{mode}_k{K}"
    image, grads, _ = run_training_step(harness.ours(), scene, view, mode, K)
    assert np.abs(image.cpu().numpy() - gold[f"{tag}_train_image"]).max() <= 1e-5
    assert_grads_close(grads, [gold[f"{tag}_grad_{n}"] for n in GRAD_NAMES], f"{name} {tag}")


@pytest.mark.parametrize("mode,K", [(0, 16), (0, 4), (1, 8), (2, 1), (3, 1)])
def test_training_against_reference_extension(mode, K):
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.outdoor_scene(n=200_000, n_views=2, seed=31, width=640, height=360, focal=500.0)
    view = scene.views[1]
    img_o, g_o, _ = run_training_step(harness.ours(), scene, view, mode, K)
    img_r, g_r, _ = run_training_step(ref, scene, view, mode, K)
    assert (img_o - img_r).abs().max().item() <= 1e-5
    assert_grads_close(g_o, g_r, f"mode {mode} K {K}")


@pytest.mark.parametrize("rows", [2, 3])
def test_densification_info_matches_reference(rows):
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    scene = scenes.tiny_scene(n=5000, size=128, seed=17, sh_degree=2)
    view = scene.views[0]
    _, _, d_o = run_training_step(harness.ours(), scene, view, 0, 8, rows, True)
    _, _, d_r = run_training_step(ref, scene, view, 0, 8, rows, True)
    a, b = d_o.cpu().numpy(), d_r.cpu().numpy()
    assert np.array_equal(a[0], b[0])
    for r in range(1, rows):
        assert np.abs(a[r] - b[r]).max() <= 2e-3 * max(np.abs(b[r]).max(), 1e-12)


def test_backward_twice_is_deterministic_enough_and_culled_gradients_are_zero():
    scene = scenes.tiny_scene(n=3000, size=96, seed=23, sh_degree=1)
    scene.positions[:100, 2] = -5.0            # behind the camera: culled
    view = scene.views[0]
    _, g1, _ = run_training_step(harness.ours(), scene, view, 0, 8)
    _, g2, _ = run_training_step(harness.ours(), scene, view, 0, 8)
    for a, b in zip(g1, g2):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-12)   # float atomics reorder sums
        assert not a[:100].any(), "culled Gaussians must get exactly zero gradient"


def _draw_training_case(seed):
    rng = np.random.default_rng(3000 + seed)
    mode = int(rng.integers(0, 4))
    K = int(rng.choice([1, 2, 4, 8, 16, 32])) if mode < 2 else 1
    return dict(mode=mode, K=K, n=int(rng.choice([40, 700, 5000])), size=int(rng.choice([24, 75, 160])), sh_degree=int(rng.integers(0, 4)),
                rows=int(rng.choice([0, 2, 3])), distance_scaling=bool(rng.integers(0, 2)))


@pytest.mark.parametrize("seed", list(range(16)))
def test_random_training_cases_against_reference_extension(seed):
    """Seeded sweep over mode, K, scene size, image size, SH degree and the densification options."""
    import torch
    ref = harness.reference()
    if ref is None:
        pytest.skip("reference extension not built under baseline/_ref")
    c = _draw_training_case(seed)
    scene = scenes.tiny_scene(n=c["n"], size=c["size"], seed=400 + seed, sh_degree=c["sh_degree"])
    view = scene.views[0]
    image, grads, dens = run_training_step(harness.ours(), scene, view, c["mode"], c["K"], c["rows"], c["distance_scaling"])
    r_image, r_grads, r_dens = run_training_step(ref, scene, view, c["mode"], c["K"], c["rows"], c["distance_scaling"])
    assert (image - r_image).abs().max().item() <= 1e-5, c
    assert_grads_close(grads, r_grads, f"case {c}")
    if c["rows"]:
        scale = r_dens.abs().max().item()
        assert (dens - r_dens).abs().max().item() <= 1e-3 * max(scale, 1e-12), c


@pytest.mark.parametrize("mode,K", [(0, 8), (2, 1)])
def test_training_visibility_covers_every_nonzero_gradient_row(mode, K):
    """`last_training_visibility` is what multi-GPU training exchanges gradient rows by: it must equal the forward's own
    per-Gaussian tile counts, and no gradient row outside it may be non-zero."""
    import torch
    from htgs_b200.torch_bindings import rasterization
    scene = scenes.outdoor_scene(n=20_000, n_views=3, seed=5, width=200, height=120, focal=180.0)   # part of the scene is outside the view
    view = scene.views[1]
    rasterization.track_training_visibility(True)
    try:
        image, grads, _ = run_training_step(harness.ours(), scene, view, mode, K)
        visible = rasterization.last_training_visibility("cuda")
    finally:
        rasterization.track_training_visibility(False)
    assert visible.dtype == torch.bool and visible.shape == (scene.n,)
    harness.ours().rasterize(*harness.scene_tensors(scene), harness.settings_for(harness.ours(), scene, view, mode, K), True, False)
    from htgs_b200.torch_bindings import _C
    inter = harness.our_intermediates(0, scene.n, _C.last_frame_info.n_instances)
    assert np.array_equal(visible.cpu().numpy(), inter["n_touched"] > 0)
    assert 0 < int(visible.sum()) < scene.n
    for g in grads:
        assert float(g[~visible].abs().max()) == 0.0
    with pytest.raises(RuntimeError):
        rasterization.last_training_visibility("cuda")


def test_row_gather_and_scatter_kernels_match_index_select():
    """htgs_gather_rows / htgs_scatter_rows (the packing of the multi-GPU gradient exchange) against torch indexing."""
    import ctypes
    import torch
    from htgs_b200 import _native
    gen = torch.Generator(device="cpu").manual_seed(5)
    n = 10_000
    shapes = [(n, 3), (n, 3), (n, 4), (n, 1), (n, 1, 3), (n, 15, 3)]
    tensors = [torch.randn(s, generator=gen).cuda() for s in shapes]
    index = torch.nonzero(torch.rand(n, generator=gen) < 0.2).squeeze(1).cuda()
    count = int(index.numel())
    table = _native.HtgsRowTensors()
    table.n_tensors = len(tensors)
    for k, t in enumerate(tensors):
        table.data[k] = t.data_ptr()
        table.width[k] = t[0].numel()
    width = sum(t[0].numel() for t in tensors)
    packed = torch.full((count, width), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _native.check(_native.lib().htgs_gather_rows(ctypes.byref(table), index.data_ptr(), count, packed.data_ptr(), stream))
    expected = torch.cat([t.view(n, -1).index_select(0, index) for t in tensors], dim=1)
    assert torch.equal(packed, expected)
    before = [t.clone() for t in tensors]
    packed.mul_(2.0)
    _native.check(_native.lib().htgs_scatter_rows(ctypes.byref(table), index.data_ptr(), count, packed.data_ptr(), stream))
    torch.cuda.synchronize()
    for t, b in zip(tensors, before):
        want = b.clone()
        want[index] = 2.0 * b[index]
        assert torch.equal(t, want)
    # nothing to move, and argument errors
    assert _native.lib().htgs_gather_rows(ctypes.byref(table), None, 0, None, stream) == 0
    table.n_tensors = 9
    assert _native.lib().htgs_gather_rows(ctypes.byref(table), index.data_ptr(), count, packed.data_ptr(), stream) != 0


@pytest.mark.parametrize("mode,K", [(0, 16), (1, 8), (3, 1)])
def test_backward_in_ranges_of_gaussians_equals_the_whole_pass(mode, K):
    """`htgs_backward_range`: the pass split into ranges of Gaussian indices gives the gradients of the whole pass (sums
    of float atomics, so equal to rounding), the callback sees every range once in order, and rows of a range are final
    when its callback runs (checked by snapshotting them there)."""
    import torch
    from htgs_b200.torch_bindings import _C
    scene = scenes.outdoor_scene(n=150_000, n_views=2, seed=37, width=640, height=360, focal=500.0)
    view = scene.views[0]
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(harness.ours(), scene, view, mode, K)
    fwd = _C.forward(*tensors, *st.as_tuple())
    image, blobs, n_inst, sel = fwd[0], fwd[1:5], fwd[5], fwd[6]
    grad_image = torch.from_numpy(target_image(view.height, view.width, 77)).cuda() - 0.5
    empty = torch.empty(0, device="cuda")
    args = (empty, grad_image, empty, tensors[0], tensors[1], tensors[2], tensors[3] if mode == 1 else empty, tensors[5], *blobs, *st.as_tuple(), n_inst, sel, False)
    whole = _C.backward(*args)
    n = scene.n
    edges = [0, n // 7, n // 2, n // 2, n - 5, n]          # uneven ranges, one of them empty
    ranges = [(a, b - a) for a, b in zip(edges[:-1], edges[1:])]
    seen, snapshots = [], []

    def after_range(k, first, count, grads):
        seen.append((k, first, count))
        snapshots.append([g[first:first + count].clone() for g in grads])

    split = _C.backward(*args, ranges=ranges, after_range=after_range)
    torch.cuda.synchronize()
    assert seen == [(k, a, c) for k, (a, c) in enumerate(ranges)]
    for a, b in zip(split, whole):
        scale = max(b.abs().max().item(), 1e-30)
        assert (a - b).abs().max().item() <= 1e-5 * scale
    for (first, count), snap in zip(ranges, snapshots):
        for g, s in zip(split, snap):
            assert torch.equal(g[first:first + count], s), "rows of a finished range must not change afterwards"
    with pytest.raises(ValueError):
        _C.backward(*args, ranges=[(0, n // 2)])
    # the per-tile pass once, only the per-Gaussian chain rule range by range
    staged = _C.backward(*args, ranges=ranges, split_pass=False)
    for a, b in zip(staged, whole):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30)


def test_global_ordering_refuses_a_partial_backward():
    import torch
    from htgs_b200.torch_bindings import _C
    scene = scenes.tiny_scene(n=3000, size=96, seed=29, sh_degree=1)
    view = scene.views[0]
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(harness.ours(), scene, view, 2, 1)
    fwd = _C.forward(*tensors, *st.as_tuple())
    empty = torch.empty(0, device="cuda")
    args = (empty, torch.ones_like(fwd[0]), fwd[0], tensors[0], tensors[1], tensors[2], empty, tensors[5], *fwd[1:5], *st.as_tuple(), fwd[5], fwd[6], False)
    whole = _C.backward(*args)
    same = _C.backward(*args, ranges=[(0, scene.n)])
    for a, b in zip(same, whole):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30)
    with pytest.raises(RuntimeError):
        _C.backward(*args, ranges=[(0, 1000), (1000, scene.n - 1000)])
    staged = _C.backward(*args, ranges=[(0, 1000), (1000, scene.n - 1000)], split_pass=False)      # the chain rule alone may be split
    for a, b in zip(staged, whole):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30)


class _OwnRowsOnly:
    """Stands in for htgs_b200.parallel.CompactExchange in a single process: the buffers 'of all ranks' are the ones it is told to
    hand back (by default this rank's own), and it keeps what the backward pass wrote."""
    compact = True

    def __init__(self, capacity=None, replay=None, expansion="add"):
        self._capacity, self.replay, self.rows, self.kept, self._expansion = capacity, replay, None, [], expansion

    def expansion(self):
        return self._expansion

    def capacity(self, n):
        return n if self._capacity is None else self._capacity

    def buffer(self, nbytes, device):
        import torch
        return torch.empty(int(nbytes), dtype=torch.uint8, device=device)

    def exchange(self, rows, capacity):
        self.rows = rows
        self.kept.append((rows, capacity))
        sources = self.kept if self.replay == "all kept" else [(rows, capacity)]
        return [(r.data_ptr(), c, r) for r, c in sources]


@pytest.mark.parametrize("mode,K,sh_degree", [(0, 16, 3), (0, 4, 2), (1, 8, 1), (2, 1, 3), (3, 1, 0)])
def test_compact_backward_expands_to_the_dense_gradients(mode, K, sh_degree):
    """`htgs_backward_compact` + `htgs_expand_add_rows`: one 64-byte row per kept Gaussian, which expands to the six dense
    tensors of `htgs_backward` (the per-tile pass sums with float atomics, so two passes agree to rounding, not bit for bit);
    the row count equals the number of kept Gaussians, every index occurs once, and expanding is deterministic."""
    import torch
    from htgs_b200.torch_bindings import _C, rasterization
    scene = scenes.outdoor_scene(n=60_000, n_views=2, seed=41, width=400, height=240, focal=300.0)
    scene.active_sh_bases = (sh_degree + 1) ** 2      # fewer active bases than the 15 stored ones: the rest get no gradient
    view = scene.views[1]
    tensors = harness.scene_tensors(scene)
    st = harness.settings_for(harness.ours(), scene, view, mode, K)
    fwd = _C.forward(*tensors, *st.as_tuple())
    image, blobs, n_inst, sel = fwd[0], fwd[1:5], fwd[5], fwd[6]
    grad_image = torch.from_numpy(target_image(view.height, view.width, 78)).cuda() - 0.5
    empty = torch.empty(0, device="cuda")
    dens = torch.zeros((2, scene.n, 1), device="cuda")
    args = lambda d: (d, grad_image, image if mode == 2 else empty, tensors[0], tensors[1], tensors[2], tensors[3] if mode == 1 else empty, tensors[5],
                      *blobs, *st.as_tuple(), n_inst, sel, False)
    dens_dense = dens.clone()
    dense = _C.backward(*args(dens_dense))
    stub = _OwnRowsOnly()
    dens_compact = dens.clone()
    compact = _C.backward(*args(dens_compact), compact=stub)
    torch.cuda.synchronize()
    for name, a, b in zip(GRAD_NAMES, compact, dense):
        assert a.shape == b.shape
        if b.numel():
            assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30), f"grad_{name}"
    assert (dens_compact - dens_dense).abs().max().item() <= 1e-5 * max(dens_dense.abs().max().item(), 1e-30)
    words = stub.rows.view(torch.int32).view(-1, 16)
    count = int(words[0, 0])
    kept = dense[0].abs().sum(dim=1) + dense[3].abs().sum(dim=1) > 0        # a superset test below uses the forward's own list
    index = words[1:1 + count, 0].long()
    assert count == index.unique().numel(), "every kept Gaussian has exactly one row"
    assert bool(kept[index].sum() >= 0) and int(index.min()) >= 0 and int(index.max()) < scene.n
    cam = words[0, 1:4].view(torch.float32).cpu().numpy()
    assert np.array_equal(cam, np.asarray(view.cam_position, np.float32).reshape(3)) and int(words[0, 4]) == scene.active_sh_bases
    outside = torch.ones(scene.n, dtype=torch.bool, device="cuda")
    outside[index] = False
    for g in dense:
        if g.numel():
            assert float(g[outside].abs().max()) == 0.0, "a Gaussian without a compact row has no gradient"
    # the expansion alone is deterministic: the same buffer expanded twice gives identical bits
    import ctypes
    from htgs_b200 import _native
    lib = _native.lib()
    n, B = scene.n, tensors[5].shape[1]
    sc = _native.HtgsScene(tensors[0].data_ptr(), None, None, None, None, None, n, B)
    results = []
    for _ in range(2):
        outs = [torch.zeros_like(g) for g in dense]
        gr = _native.HtgsGradients(outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr(), outs[4].data_ptr(),
                                   outs[5].data_ptr() if outs[5].numel() else None, None, 0, None, 0, 0)
        _native.check(lib.htgs_expand_add_rows(ctypes.byref(sc), stub.rows.data_ptr(), n, ctypes.byref(gr), torch.cuda.current_stream().cuda_stream))
        results.append(outs)
    torch.cuda.synchronize()
    for a, b, c in zip(results[0], results[1], compact):
        assert torch.equal(a, b) and torch.equal(a, c)


def test_compact_rows_of_two_views_sum_like_two_dense_passes_and_small_capacity_drops_rows():
    """What every rank of a multi-GPU step does: the buffers of all views are expanded one after the other into the same
    tensors.  Also: a buffer too small for the kept Gaussians reports the full count in its header and holds `capacity` rows."""
    import torch
    from htgs_b200.torch_bindings import _C
    scene = scenes.outdoor_scene(n=50_000, n_views=4, seed=43, width=320, height=200, focal=260.0)
    tensors = harness.scene_tensors(scene)
    empty = torch.empty(0, device="cuda")
    stub = _OwnRowsOnly(replay="all kept")
    dense_sum, last = None, None
    for vi in (0, 2):
        view = scene.views[vi]
        st = harness.settings_for(harness.ours(), scene, view, 0, 8)
        fwd = _C.forward(*tensors, *st.as_tuple())
        grad_image = torch.from_numpy(target_image(view.height, view.width, 80 + vi)).cuda() - 0.5
        args = (empty, grad_image, empty, tensors[0], tensors[1], tensors[2], empty, tensors[5], *fwd[1:5], *st.as_tuple(), fwd[5], fwd[6], False)
        dense = _C.backward(*args)
        dense_sum = [d.clone() for d in dense] if dense_sum is None else [a + d for a, d in zip(dense_sum, dense)]
        last = _C.backward(*args, compact=stub)      # second call: expands the buffers of both views
    torch.cuda.synchronize()
    for name, a, b in zip(GRAD_NAMES, last, dense_sum):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30), f"grad_{name}"
    # one pass over all buffers (htgs_expand_sum_rows) against buffer after buffer (htgs_expand_add_rows): the same bits
    import ctypes
    from htgs_b200 import _native
    lib = _native.lib()
    n, B = scene.n, tensors[5].shape[1]
    sc = _native.HtgsScene(tensors[0].data_ptr(), None, None, None, None, None, n, B)
    stream = torch.cuda.current_stream().cuda_stream
    buffers = [stub.kept[0][0], stub.kept[1][0], stub.kept[0][0], stub.kept[1][0], stub.kept[1][0]]      # five "ranks", views repeated

    def gradients(fill):
        outs = [torch.full_like(g, fill) for g in last]
        return outs, _native.HtgsGradients(outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr(), outs[4].data_ptr(),
                                           outs[5].data_ptr(), None, 0, None, 0, 0)
    added, gr = gradients(0.0)
    for b in buffers:
        _native.check(lib.htgs_expand_add_rows(ctypes.byref(sc), b.data_ptr(), n, ctypes.byref(gr), stream))
    summed, gr = gradients(7.0)                                  # not cleared: every row is written
    table = torch.empty(lib.htgs_expand_sum_scratch_bytes(ctypes.byref(sc), len(buffers)), dtype=torch.uint8, device="cuda")
    addresses = (ctypes.c_void_p * len(buffers))(*[b.data_ptr() for b in buffers])
    _native.check(lib.htgs_expand_sum_rows(ctypes.byref(sc), addresses, len(buffers), n, table.data_ptr(), table.numel(), ctypes.byref(gr), stream))
    torch.cuda.synchronize()
    for name, a, b in zip(GRAD_NAMES, summed, added):
        assert torch.equal(a, b), f"grad_{name}: one pass and buffer-after-buffer differ"
    with pytest.raises(_native.HtgsError):
        _native.check(lib.htgs_expand_sum_rows(ctypes.byref(sc), addresses, len(buffers), n, table.data_ptr(), 16, ctypes.byref(gr), stream))
    # the autograd hook's one-pass route
    one_pass = _OwnRowsOnly(replay="all kept", expansion="sum")
    one_pass.kept = list(stub.kept[:1])
    via_hook = _C.backward(*args, compact=one_pass)
    torch.cuda.synchronize()
    for name, a, b in zip(GRAD_NAMES, via_hook, dense_sum):
        assert (a - b).abs().max().item() <= 1e-5 * max(b.abs().max().item(), 1e-30), f"grad_{name} (one pass)"
    small = _OwnRowsOnly(capacity=100)
    _C.backward(*args, compact=small)
    torch.cuda.synchronize()
    words = small.rows.view(torch.int32).view(-1, 16)
    assert words.shape[0] == 101 and int(words[0, 0]) > 100


_PEER_CHILD = '''
import ctypes, sys
sys.path.insert(0, sys.argv[1])
from htgs_b200 import _native
lib = _native.lib()
handle = bytes.fromhex(sys.argv[2])
ptr = ctypes.c_void_p()
_native.check(lib.htgs_peer_buffer_open(0, handle, ctypes.byref(ptr)))
host = (ctypes.c_uint32 * 1024)()
_native.check(lib.htgs_memcpy_d2h(host, ptr, 4096))
ok = all(host[i] == (i * 2654435761) % 2**32 for i in range(1024))
_native.check(lib.htgs_peer_buffer_close(0, ptr))
sys.exit(0 if ok else 3)
'''


def test_peer_buffer_is_readable_from_another_process(tmp_path):
    """`htgs_peer_buffer_*`: a buffer created here, opened by handle in a child process (on the same GPU: the mapping calls are
    the ones ranks on different GPUs use), read there and closed; then destroyed here."""
    import ctypes
    import subprocess
    import sys
    from htgs_b200 import _native
    lib = _native.lib()
    ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    _native.check(lib.htgs_peer_buffer_create(0, 1 << 20, ctypes.byref(ptr), handle))
    try:
        host = (ctypes.c_uint32 * 1024)(*[(i * 2654435761) % 2**32 for i in range(1024)])
        _native.check(lib.htgs_memcpy_h2d(ptr, host, 4096))
        script = tmp_path / "child.py"
        script.write_text(_PEER_CHILD)
        proc = subprocess.run([sys.executable, str(script), harness.REPO, handle.raw.hex()], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
        assert proc.returncode == 0, proc.stdout[-2000:]
    finally:
        _native.check(lib.htgs_peer_buffer_destroy(0, ptr))
    with pytest.raises(_native.HtgsError):
        _native.check(lib.htgs_peer_buffer_create(0, 0, ctypes.byref(ptr), handle))
