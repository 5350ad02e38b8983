"""Makes tests/golden/ops_golden.json: the outputs of the reference's own host functions for the per-layer
operations (cpu_ops.h:12-28) at the sizes of the tests' tiny models A and B (head sizes 16 and 32, 4:2 and 3:1
heads, rotary bases 1e4 and 1e6, positions 0, 1, 63 and 200), from ops_driver.cpp linked against the reference's
libfriday_engine.a (built as make_golden.py says).  tests/test_golden.py repeats the driver's input generator and
compares the plain implementation's functions with these outputs; the reference rounds every output to fp16, so the
agreement is to about 1e-3 relative.

    python tests/golden/make_ops_golden.py <reference dir> <build dir>
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main(reference_dir, build_dir):
    exe = os.path.join(build_dir, "ops_driver")
    subprocess.run(["g++", "-O2", "-std=c++17", "-DFRIDAY_HAVE_CUDA=0", "-I", reference_dir, "-I",
                    os.path.join(reference_dir, "include"), os.path.join(HERE, "ops_driver.cpp"),
                    os.path.join(build_dir, "libfriday_engine.a"), "-lpthread", "-o", exe], check=True)
    out = subprocess.run([exe], check=True, stdout=subprocess.PIPE, text=True).stdout
    with open(os.path.join(HERE, "ops_golden.json"), "w") as f:
        f.write(out)
    print("wrote ops_golden.json (%d bytes)" % len(out))


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
