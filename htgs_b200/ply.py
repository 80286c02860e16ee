"""3D-Gaussian-splatting `.ply` files as the reference writes them (Model.py:404-435 `as_ply_dict`): one `vertex`
element of float32 properties

    x y z | f_dc_0..2 | f_rest_0..3B-1 | opacity | scale_0..2 | rot_0..3

with the SH coefficients stored channel-major (`[N,B,3].transpose(1,2).flatten(1)`), opacities as logits and scales as
logs ("pre-activation", what most viewers expect) and rotations as (r, x, y, z).  Pure numpy; binary little-endian and
ASCII files are read, binary little-endian is written.
"""
from __future__ import annotations

from typing import Dict

import numpy as np

_PLY_TYPES = {"char": "i1", "int8": "i1", "uchar": "u1", "uint8": "u1", "short": "i2", "int16": "i2", "ushort": "u2", "uint16": "u2",
              "int": "i4", "int32": "i4", "uint": "u4", "uint32": "u4", "float": "f4", "float32": "f4", "double": "f8", "float64": "f8"}


def property_names(n_rest_bases: int):
    return (["x", "y", "z"] + ["f_dc_0", "f_dc_1", "f_dc_2"] + [f"f_rest_{i}" for i in range(3 * n_rest_bases)] + ["opacity"]
            + ["scale_0", "scale_1", "scale_2"] + ["rot_0", "rot_1", "rot_2", "rot_3"])


def write_ply(path: str, positions, sh_0, sh_rest, raw_opacities, raw_scales, rotations) -> None:
    """positions [N,3], sh_0 [N,1,3], sh_rest [N,B,3], raw_opacities [N,1] (logits), raw_scales [N,3] (logs), rotations [N,4]."""
    positions = np.asarray(positions, np.float32)
    n = positions.shape[0]
    sh_0 = np.asarray(sh_0, np.float32).reshape(n, 1, 3)
    sh_rest = np.asarray(sh_rest, np.float32)
    n_rest = sh_rest.shape[1] if sh_rest.ndim == 3 else (sh_rest.size // (3 * n) if n else 0)
    sh_rest = sh_rest.reshape(n, n_rest, 3)
    attributes = np.concatenate((positions.reshape(n, 3), sh_0.transpose(0, 2, 1).reshape(n, 3), sh_rest.transpose(0, 2, 1).reshape(n, 3 * n_rest),
                                 np.asarray(raw_opacities, np.float32).reshape(n, 1), np.asarray(raw_scales, np.float32).reshape(n, 3),
                                 np.asarray(rotations, np.float32).reshape(n, 4)), axis=1)
    names = property_names(n_rest)
    header = ["ply", "format binary_little_endian 1.0", f"element vertex {n}"] + [f"property float {name}" for name in names] + ["end_header"]
    with open(path, "wb") as f:
        f.write(("\n".join(header) + "\n").encode("ascii"))
        f.write(np.ascontiguousarray(attributes, dtype="<f4").tobytes())


def _read_header(f):
    if f.readline().strip() != b"ply":
        raise ValueError("not a ply file")
    fmt, elements, current = None, [], None
    while True:
        line = f.readline()
        if not line:
            raise ValueError("ply header is not terminated")
        tok = line.decode("ascii", "replace").split()
        if not tok or tok[0] == "comment" or tok[0] == "obj_info":
            continue
        if tok[0] == "format":
            fmt = tok[1]
        elif tok[0] == "element":
            current = {"name": tok[1], "count": int(tok[2]), "properties": []}
            elements.append(current)
        elif tok[0] == "property":
            if tok[1] == "list":
                raise ValueError("list properties are not supported")
            if tok[1] not in _PLY_TYPES:
                raise ValueError(f"unknown ply property type {tok[1]}")
            current["properties"].append((tok[2], _PLY_TYPES[tok[1]]))
        elif tok[0] == "end_header":
            break
    if fmt not in ("binary_little_endian", "binary_big_endian", "ascii"):
        raise ValueError(f"unsupported ply format {fmt}")
    return fmt, elements


def read_ply(path: str) -> Dict[str, np.ndarray]:
    """Returns float32 arrays: positions [N,3], sh_0 [N,1,3], sh_rest [N,B,3], raw_opacities [N,1], raw_scales [N,3],
    rotations [N,4] (as stored: not normalised).  Properties are looked up by name, so extra ones (normals) are ignored."""
    with open(path, "rb") as f:
        fmt, elements = _read_header(f)
        vertex = None
        for el in elements:
            if fmt == "ascii":
                rows = [f.readline().split() for _ in range(el["count"])]
                data = np.zeros(el["count"], dtype=[(n, t) for n, t in el["properties"]])
                for c, (n, t) in enumerate(el["properties"]):
                    data[n] = np.array([r[c] for r in rows], dtype=np.float64).astype(t) if rows else np.zeros(0, t)
            else:
                order = "<" if fmt == "binary_little_endian" else ">"
                dtype = np.dtype([(n, order + t) for n, t in el["properties"]])
                raw = f.read(dtype.itemsize * el["count"])
                if len(raw) != dtype.itemsize * el["count"]:
                    raise ValueError("ply file is truncated")
                data = np.frombuffer(raw, dtype=dtype, count=el["count"])
            if el["name"] == "vertex":
                vertex = data
        if vertex is None:
            raise ValueError("ply file has no vertex element")
    names = vertex.dtype.names

    def cols(keys):
        missing = [k for k in keys if k not in names]
        if missing:
            raise ValueError(f"ply file lacks properties {missing}")
        return np.stack([vertex[k].astype(np.float32) for k in keys], axis=1) if keys else np.zeros((vertex.shape[0], 0), np.float32)

    n = vertex.shape[0]
    n_rest_values = sum(1 for k in names if k.startswith("f_rest_"))
    if n_rest_values % 3:
        raise ValueError("number of f_rest_ properties is not a multiple of 3")
    n_rest = n_rest_values // 3
    return {
        "positions": cols(["x", "y", "z"]),
        "sh_0": cols(["f_dc_0", "f_dc_1", "f_dc_2"]).reshape(n, 3, 1).transpose(0, 2, 1).copy(),
        "sh_rest": cols([f"f_rest_{i}" for i in range(n_rest_values)]).reshape(n, 3, n_rest).transpose(0, 2, 1).copy(),
        "raw_opacities": cols(["opacity"]),
        "raw_scales": cols(["scale_0", "scale_1", "scale_2"]),
        "rotations": cols(["rot_0", "rot_1", "rot_2", "rot_3"]),
    }
