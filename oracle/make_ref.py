"""Stage the reference's own CPU code for the SBMM path under oracle/_ref/.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  The reference is Python and cannot be imported as
a package (its __init__ pulls in cupy), so the two files that hold the path are taken as
they are, by file path, from a checkout of the reference:

    deltazip/core/quant.py          Quantizer.find_params, quantize          (:9-86)
    deltazip/nn_modules/qlinear.py  QuantLinear.pack / unpack / forward      (:83-341)

    python oracle/make_ref.py [/path/to/deltazip-checkout]

oracle/_ref/ is excluded from version control (the files are the reference's, not this
project's) but travels with the working tree to the machine that runs the benchmark, where
`oracle/reference_path.py` loads them so that the timed CPU baseline is the reference's own
code (`cpu_baseline.kind == "reference"`).  When oracle/_ref/ is absent the baseline falls
back to the restatement in oracle/torch_port.py (`kind == "port"`).
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = {"deltazip/core/quant.py": "quant.py", "deltazip/nn_modules/qlinear.py": "qlinear.py"}


def stage(checkout: str) -> bool:
    """Copies the files; returns False (and changes nothing) when the checkout lacks them."""
    srcs = {os.path.join(checkout, rel): name for rel, name in FILES.items()}
    if not all(os.path.isfile(s) for s in srcs):
        return False
    os.makedirs(DEST, exist_ok=True)
    for src, name in srcs.items():
        shutil.copyfile(src, os.path.join(DEST, name))
    with open(os.path.join(DEST, "README"), "w") as fh:
        fh.write("Unmodified files of eth-easl/deltazip staged by oracle/make_ref.py; not part of "
                 "this project's sources.\n")
    return True


if __name__ == "__main__":
    path = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    ok = stage(path)
    print("staged" if ok else f"no reference checkout at {path}", DEST)
    sys.exit(0 if ok else 1)
