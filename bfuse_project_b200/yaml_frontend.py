"""The reference's on-disk interface: read its `kernels.yaml` / `fusions.yaml`, plan every listed pair
with this runtime's host scheduler and write the fused-kernel records in the schema of its
`bfuse_kernels.yaml` / `hfuse_kernels.yaml`, so that the reference's own tooling can consume them.

Schemas (horizontal-fuser/include/fuse/Utils.h:69-112): `kernels.yaml` maps a name to
{KernelName, HasBarriers, GridDim{X,Y,Z}, BlockDim{X,Y,Z}, Reg, ExecTime (optional, default -1)};
`fusions.yaml` is a list of {File, Kernels: [k1, k2]}; the output maps `<k1>_<k2>_fused_{bfuse,hfuse}`
(src/Contexts.cc:67-84) to a kernel record with the fused dims, HasBarriers true, Reg 32 and
ExecTime left at its default (src/Fuse.cc:203-220, 358-375).

    python -m bfuse_project_b200.yaml_frontend [-b] [-y out_dir] fusions.yaml kernels.yaml

`-b` selects block-level fusion (the zig-zag 1:1 pattern the reference uses), without it the
thread-level split -- the meaning of the reference fuser's own `-b` switch.  No GPU is needed.
"""
import argparse
import os
import sys

import yaml

from . import THREAD_SPLIT, ZIGZAG, Plan


def load_kernels(path):
    """{name: {"KernelName", "HasBarriers", "GridDim": (x, y, z), "BlockDim": (x, y, z), "Reg", "ExecTime"}}."""
    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    out = {}
    for name, rec in raw.items():
        for key in ("KernelName", "HasBarriers", "GridDim", "BlockDim", "Reg"):
            if key not in rec:
                raise ValueError("%s: kernel %s has no %s" % (path, name, key))
        out[name] = {"KernelName": rec["KernelName"], "HasBarriers": bool(rec["HasBarriers"]),
                     "GridDim": tuple(int(rec["GridDim"][a]) for a in "XYZ"),
                     "BlockDim": tuple(int(rec["BlockDim"][a]) for a in "XYZ"),
                     "Reg": int(rec["Reg"]), "ExecTime": float(rec.get("ExecTime", -1))}
    return out


def load_fusions(path):
    """[(file, [kernel names])] in file order."""
    with open(path) as f:
        raw = yaml.safe_load(f) or []
    out = []
    for i, rec in enumerate(raw):
        if "File" not in rec or "Kernels" not in rec:
            raise ValueError("%s: entry %d needs File and Kernels" % (path, i))
        if len(rec["Kernels"]) != 2:
            raise ValueError("%s: entry %d: exactly two kernels per fusion" % (path, i))
        out.append((rec["File"], list(rec["Kernels"])))
    return out


def fuse_records(kernels, fusions, block_level=True, pattern=None, param_m=1, param_n=1):
    """{fused name: record} for every listed pair; records carry the fused GridDim / BlockDim."""
    pattern = (ZIGZAG if block_level else THREAD_SPLIT) if pattern is None else pattern
    suffix = "_fused_hfuse" if pattern == THREAD_SPLIT else "_fused_bfuse"
    out = {}
    for _, names in fusions:
        for n in names:
            if n not in kernels:
                raise KeyError("fusion refers to unknown kernel %s" % n)
        dims = [list(kernels[n]["GridDim"]) + list(kernels[n]["BlockDim"]) for n in names]
        plan = Plan(dims, pattern, param_m, param_n)
        # the fused name is built from the kernels.yaml map keys listed in the fusion, not from the KernelName
        # fields (horizontal-fuser/src/Contexts.cc:67-84: FusedKernelName += KName + '_')
        name = "_".join(names) + suffix
        out[name] = {"KernelName": name, "HasBarriers": True, "GridDim": plan.fused_grid, "BlockDim": plan.fused_block,
                     "Reg": 32, "ExecTime": -1.0}
    return out


def dump_kernels(records, path):
    """Write records in the reference's output schema (ExecTime omitted at its default, as llvm::yaml does)."""
    doc = {}
    for name, r in sorted(records.items()):   # the reference keeps its records in a std::map: written sorted by name
        e = {"KernelName": r["KernelName"], "HasBarriers": bool(r["HasBarriers"]),
             "GridDim": dict(zip("XYZ", (int(v) for v in r["GridDim"]))),
             "BlockDim": dict(zip("XYZ", (int(v) for v in r["BlockDim"]))), "Reg": int(r["Reg"])}
        if r.get("ExecTime", -1) != -1:
            e["ExecTime"] = float(r["ExecTime"])
        doc[name] = e
    with open(path, "w") as f:
        f.write("---\n")
        yaml.safe_dump(doc, f, sort_keys=False, default_flow_style=False)
        f.write("...\n")


def main(argv=None):
    """Same switches and argument order as the reference fuser (horizontal-fuser/src/main.cc:20-70):
    [-b] [-y yaml_output_dir] fusion_config kernel_config [compile_commands]; the record file is
    `bfuse_kernels.yaml` or `hfuse_kernels.yaml` in the output directory.  `-o` (rewritten sources) and
    compile_commands are accepted and ignored: there are no sources to rewrite."""
    ap = argparse.ArgumentParser(prog="yaml_frontend", description="plan the pairs of a fusion config and write the fused-kernel records")
    ap.add_argument("-b", action="store_true", help="block-level fusion (default: thread-level)")
    ap.add_argument("-y", default=".", metavar="yaml_output", help="directory for the record file (default: .)")
    ap.add_argument("-o", default=".", metavar="output", help="accepted for compatibility, unused")
    ap.add_argument("fusion_config")
    ap.add_argument("kernel_config")
    ap.add_argument("compile_commands", nargs="?", help="accepted for compatibility, unused")
    args = ap.parse_args(argv)
    out = os.path.join(args.y, "bfuse_kernels.yaml" if args.b else "hfuse_kernels.yaml")
    try:
        recs = fuse_records(load_kernels(args.kernel_config), load_fusions(args.fusion_config), block_level=args.b)
        dump_kernels(recs, out)
    except (OSError, ValueError, KeyError, yaml.YAMLError) as e:
        print("yaml_frontend: %s" % e, file=sys.stderr)
        return 1
    print("%d fused kernels written to %s" % (len(recs), out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
