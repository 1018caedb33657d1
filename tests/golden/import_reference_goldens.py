"""Copy the reference's own golden vectors for the hot path into tests/golden/reference/.

The files are the PyTorch-generated regression data the reference's layer tests read
(test/regression_data, written by test/gen_reg_data.py with torch.manual_seed(0); format:
big-endian uint32 element count, then raw little-endian float32, test/test_utils.hpp
:187-215).  Everything up to 150 KB is taken, plus a few 96-channel 30x30 cases that give
the convolution kernels a non-trivial size and the 19x19 box-decoding case.  Run once where the reference tree is mounted:

    python tests/golden/import_reference_goldens.py /path/to/reference
"""
import os
import shutil
import sys

EXTRA = [
    "{}__conv2d_Ci96_H30_W30_k3_s1_f_Co96_{}.bin",
    "{}__conv2d_Ci96_H30_W30_k3_s2_f_Co96_{}.bin",
    "{}__dw_conv_Ci96_H30_W30_k3_s2_f_{}.bin",
    "{}__pool_Ci96_H30_W30_k3_s2_f_{}.bin",
    "{}__yolo_Ci255_H19_W19_k0_s0_f_{}.bin",   # box decoding (YOLOLayer), the smallest of the three cases
]


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    src = os.path.join(ref, "test", "regression_data")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference")
    os.makedirs(dst, exist_ok=True)
    names = sorted(os.listdir(src))
    extra_keys = [e.split("{}")[1] for e in EXTRA]
    n = 0
    for name in names:
        if "yolov3tiny" in name or not name.endswith(".bin"):
            continue  # whole-network vectors need the Darknet weights, which the checkout lacks
        path = os.path.join(src, name)
        small = os.path.getsize(path) <= 150 * 1024
        extra = any(k in name for k in extra_keys)
        if small or extra:
            shutil.copyfile(path, os.path.join(dst, name))
            n += 1
    print(f"copied {n} files to {dst}")


if __name__ == "__main__":
    main()
