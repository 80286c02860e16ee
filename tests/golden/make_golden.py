"""Generates the golden fixtures under tests/golden/ by running the UNMODIFIED reference
extension (built under baseline/_ref/HTGSCudaBackend) on a B200:

    python tests/golden/make_golden.py            # on a machine with a GPU and the reference built

The reference ships no tests or golden vectors of its own, so these outputs of the reference
itself are what pins the CPU oracle and the CUDA path.  Inputs are not stored: they are
regenerated from the seeds in `CASES` by htgs_b200.scenes (numpy PCG64), and a SHA-256 of the
inputs is stored with every case so that a drifting generator is detected.

Per case and blend mode the file holds: the `rasterize` image and depth, the tile boxes and
tile counts of the preprocess, the sorted instance list and tile ranges (parsed from the
scratch blobs `_C.forward` returns), the training-forward image, the six gradients of
`diff_rasterize` for an L1 loss against a seeded target, the `update_max_weights` result and the `fast_rasterize` image.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import harness  # noqa: E402
from htgs_b200 import scenes  # noqa: E402

# name -> (constructor kwargs, list of (mode, K), store full images?)
CASES = {
    "small": dict(kwargs=dict(n=2048, size=96, seed=11, sh_degree=1), modes=[(0, 4), (1, 4), (2, 4), (3, 4)]),
    "small_sh3": dict(kwargs=dict(n=1024, size=64, seed=12, sh_degree=3), modes=[(0, 8), (3, 8)]),
    "config0": dict(kwargs=dict(n=16384, size=256, seed=0, sh_degree=0), modes=[(0, 16)]),
}


MAX_WEIGHT_THRESHOLD = 0.02


def inputs_digest(scene) -> str:
    h = hashlib.sha256()
    for a in scene.arrays():
        h.update(np.ascontiguousarray(a).tobytes())
    v = scene.views[0]
    for a in (v.M, v.VPM, v.cam_position):
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def target_image(height, width, seed):
    return np.random.default_rng(seed).random((3, height, width), dtype=np.float32)


def main():
    import torch
    ref = harness.reference()
    if ref is None:
        raise SystemExit("reference extension not built under baseline/_ref")
    from HTGSCudaBackend import _C as RC
    for name, case in CASES.items():
        scene = scenes.tiny_scene(**case["kwargs"])
        view = scene.views[0]
        out = {"inputs_sha256": np.frombuffer(bytes.fromhex(inputs_digest(scene)), np.uint8)}
        for mode, K in case["modes"]:
            tag = f"m{mode}_k{K}"
            tensors = harness.scene_tensors(scene)
            st = harness.settings_for(ref, scene, view, mode, K)
            for median in (False, True):
                img, depth = ref.rasterize(*tensors, st, True, median)
                out[f"{tag}_image" + ("_median" if median else "")] = img.cpu().numpy()
                out[f"{tag}_depth" + ("_median" if median else "")] = depth.cpu().numpy()
            # the reference's relaxed-precision path (fast-math build; HYBRID keeps a half-precision K-buffer): RGB only
            out[f"{tag}_fast_image"] = ref.fast_rasterize(*tensors, st, True).cpu().numpy()
            fwd = RC.forward(*tensors, *st.as_tuple())
            torch.cuda.synchronize()
            _, pp, pt, pi, _, n_inst, sel = fwd
            tw, th = (16, 16) if mode == scenes.ALPHA_BLEND_GLOBAL_ORDERING else (8, 8)
            n_tiles = ((view.width + tw - 1) // tw) * ((view.height + th - 1) // th)
            rp = harness.parse_ref_per_primitive(pp.cpu().numpy(), scene.n, mode)
            rinst = harness.parse_ref_per_instance(pi.cpu().numpy(), n_inst, harness.sort_key_bytes(mode, n_tiles), sel)
            out[f"{tag}_n_touched"] = rp["n_touched"].astype(np.uint16)
            out[f"{tag}_bounds"] = rp["bounds"].astype(np.uint16) * (rp["n_touched"][:, None] > 0)
            out[f"{tag}_sorted_prims"] = rinst["prims_sorted"].astype(np.uint32)
            out[f"{tag}_sorted_keys"] = rinst["keys_sorted"].astype(np.uint64)
            out[f"{tag}_ranges"] = harness.parse_ref_per_tile(pt.cpu().numpy(), n_tiles).astype(np.uint32)
            # training forward + backward (L1 against a seeded target, mean reduction)
            leaves = [t.clone().requires_grad_(True) for t in tensors]
            image = ref.diff_rasterize(*leaves, torch.empty(0, device="cuda"), st, False)
            target = torch.from_numpy(target_image(view.height, view.width, 1000 + mode)).cuda()
            loss = (image - target).abs().mean()
            loss.backward()
            out[f"{tag}_train_image"] = image.detach().cpu().numpy()
            for gname, leaf in zip(("positions", "scales", "rotations", "opacities", "sh_0", "sh_rest"), leaves):
                out[f"{tag}_grad_{gname}"] = leaf.grad.cpu().numpy()
            # importance weights (update_max_weights), threshold 0.02
            max_weights = torch.zeros((scene.n, 1), device="cuda")
            ref.update_max_weights(max_weights, *tensors[:4], st, MAX_WEIGHT_THRESHOLD)
            out[f"{tag}_max_weights"] = max_weights.cpu().numpy()
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(name, "->", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
