"""Builds the reference's own CUDA kernels of the UVU convolution for sm_100, as a GPU-side checker.

Test infrastructure, not product code: nothing in the package imports this file or what it builds.

The reference (LunaEquivariance v0.3.0) has no source files for its kernels: Python functions emit CUDA C++ as
strings (``src/lunatp/uvu_conv/kernels/forward.py:108`` ``make_uvu_conv_fwd_source``,
``kernels/backward.py:66`` ``make_uvu_conv_bwd_source``) and ``load_tp_extension`` (``src/utils/extension.py:38-70``)
compiles them with nvcc through ``torch.utils.cpp_extension``.  The generators and the compiler run without a GPU, so
this recipe

1. imports the reference from the checkout given on the command line (through a stub parent package, because the
   package's ``__init__`` needs e3nn),
2. lets the reference generate and compile its forward and backward extensions for a few configurations, with
   ``TORCH_CUDA_ARCH_LIST=10.0`` (the arch the reference itself would resolve on a B200: it asks torch for the visible
   device's compute capability, ``src/utils/jit.py:154-157``),
3. copies the resulting ``.so`` files to ``oracle/_ref/`` and writes ``oracle/_ref/manifest.json`` with the few
   launch facts a caller needs (which graph tables the extension wants, how many partial slabs, and up to which
   node and edge counts the extension's 32-bit index variant is valid: beyond them the reference switches to its
   64-bit variant, ``src/lunatp/utils/layout.py:441-517``).

No reference source is copied into this repository; the generated ``.cu`` text stays in the build folder under
``oracle/_ref/build`` (ignored by git and not shipped to the GPU box).  ``oracle/ref_kernels.py`` loads the libraries
on a machine with a GPU and calls their entry points.

    python oracle/build_ref.py /path/to/LunaEquivariance [config ...]
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# name -> (irreps_in1, irreps_in2, irreps_out, instructions or None for every parity-allowed uvu path, dtype names)
CONFIGS = {
    "fixture": ("32x0e+32x1o", "1x0e+1x1o", "32x0e+32x1o", None, ("float32", "float64")),
    "cfg1": ("32x1o", "1x1o", "32x0e", [(0, 0, 0, "uvu", True)], ("float64",)),
    "cfg2": ("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e+128x3o", None,
             ("float32", "float64")),
    "cfg5": ("64x0e+64x1o+64x2e", "1x0e+1x1o+1x2e", "64x0e+64x1o+64x2e", None, ("float32",)),
}


def import_reference(root: str) -> None:
    package = types.ModuleType("LunaEquivariance")
    package.__path__ = [os.path.join(root, "src")]
    sys.modules["LunaEquivariance"] = package


def main(argv) -> int:
    if len(argv) < 2:
        print(__doc__)
        return 2
    root = argv[1]
    wanted = argv[2:] or list(CONFIGS)
    os.makedirs(os.path.join(OUT, "build"), exist_ok=True)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    os.environ["LUNAEQ_CACHE_DIR"] = os.path.join(OUT, "build")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))

    import torch

    import_reference(root)
    # load_tp_extension refuses to compile without a visible device; compiling needs none.
    torch.cuda.is_available = lambda: True
    from LunaEquivariance.lunatp.utils.layout import TensorProductConfig, TensorProductPaths, configure_indexing
    from LunaEquivariance.lunatp.uvu_conv.kernels import backward as ref_backward
    from LunaEquivariance.lunatp.uvu_conv.kernels.utils import build_uvu_conv_metadata, configure_uvu_conv
    from LunaEquivariance.o3.irreps import Irreps
    from LunaEquivariance.utils.extension import load_tp_extension

    manifest_path = os.path.join(OUT, "manifest.json")
    manifest = {}
    if os.path.exists(manifest_path):
        with open(manifest_path) as handle:
            manifest = json.load(handle)

    def keep(module, target_name):
        path = module.__file__
        target = os.path.join(OUT, target_name)
        shutil.copyfile(path, target)
        return os.path.basename(target), module.__name__.split(".")[0]

    for name in wanted:
        in1, in2, out, instructions, dtypes = CONFIGS[name]
        if instructions is None:
            a, b, c = Irreps(in1), Irreps(in2), Irreps(out)
            instructions = [(i, j, k, "uvu", True) for i, (_, ia) in enumerate(a) for j, (_, ib) in enumerate(b)
                            for k, (_, ic) in enumerate(c) if ic in ia * ib]
        for dtype_name in dtypes:
            key = f"{name}.{dtype_name}"
            dtype = getattr(torch, dtype_name)
            tp = TensorProductPaths.from_tensor_product(
                TensorProductConfig(in1, in2, out, instructions, shared_weights=False, internal_weights=False))
            meta = build_uvu_conv_metadata(tp, dtype)
            digest = hashlib.sha256(json.dumps(meta, sort_keys=True, default=str).encode()).hexdigest()[:16]
            entry = manifest.get(key)
            if entry and entry.get("meta_digest") == digest and all(
                    os.path.exists(os.path.join(OUT, entry[k]["file"])) for k in ("forward", "backward")):
                if "index_edge_limit" not in entry:  # limits of the 32-bit index variant, from the reference's rule
                    probe = types.SimpleNamespace()
                    configure_indexing(probe, meta, "uvu_conv", 32)
                    entry.update(index_node_limit=int(probe.index_node_limit),
                                 index_edge_limit=int(probe.index_edge_limit))
                    with open(manifest_path, "w") as handle:
                        json.dump(manifest, handle, indent=1, sort_keys=True)
                print(f"{key}: up to date")
                continue
            print(f"{key}: building forward", flush=True)
            op = types.SimpleNamespace()
            configure_uvu_conv(op, meta, dtype, 32)  # compiles the forward extension, as the reference does
            fwd_file, fwd_module = keep(op.fwd_ext, f"{name}_{dtype_name}_fwd.so")
            print(f"{key}: building backward", flush=True)
            source, segmented, partials, vectorized, zero_x, zero_y = ref_backward.make_uvu_conv_bwd_source(
                op, with_env=False, need_grad_env=False, with_l0=False)
            bwd_name = "lunatp_uvuconv_bwd_source_fp64" if dtype == torch.float64 else "lunatp_uvuconv_bwd_source_fp32"
            bwd_ext = load_tp_extension(bwd_name, source, max_channels=op.max_channels, index_bits=op.index_bits)
            bwd_file, bwd_module = keep(bwd_ext, f"{name}_{dtype_name}_bwd.so")
            streams = getattr(bwd_ext, "_Streams", None)
            manifest[key] = dict(
                meta_digest=digest, dtype=dtype_name, irreps=[in1, in2, out],
                instructions=[list(i) for i in instructions],
                in1_dim=op.in1_dim, in2_dim=op.in2_dim, out_dim=op.out_dim, weight_numel=op.weight_numel,
                index_node_limit=int(op.index_node_limit), index_edge_limit=int(op.index_edge_limit),
                forward=dict(file=fwd_file, module=fwd_module, output_needs_zero=bool(op.forward_output_needs_zero),
                             degree_tiers=bool(op.forward_degree_tiers)),
                backward=dict(file=bwd_file, module=bwd_module, segmented=bool(segmented), partials=int(partials),
                              vectorized=bool(vectorized), zero_x=bool(zero_x), zero_y=bool(zero_y),
                              stream_count=int(streams.stream_count) if streams is not None else 0,
                              stream_priority=int(streams.stream_priority) if streams is not None else 0),
            )
            with open(manifest_path, "w") as handle:
                json.dump(manifest, handle, indent=1, sort_keys=True)
    print("manifest:", manifest_path)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
