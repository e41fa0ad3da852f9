"""Generates a training project with the reference's own TrainLib_Deployer, unmodified, and records what the reference
library makes of it.  TEST INFRASTRUCTURE: the product never reads any of this.

    python oracle/deployer_project.py [path of the reference checkout]

writes oracle/_ref/deployer/<name>/ (git-ignored; it travels to the GPU machine with the built libraries):

    main.c net.c net.h stats.h Makefile      as the Deployer writes them (tools/TrainLib_Deployer/deployer_utils)
    io_data.h init-defines.h                 written by the project's own utils/GM.py (PyTorch golden model)
    reference_run.txt                        stdout of the project linked against the reference's C sources
                                             (oracle/_ref/libpulp_ref.so) and run on this host.  The reference's fp32
                                             Linear forward drops its bias (lib/sources/pulp_linear_fp32.c:39-55: the
                                             worker it forks never reads matMul_args.bias), so that run does NOT pass
                                             the project's own check against the golden model; it is kept as a record.
                                             The acceptance test of a generated project is the project's own: the
                                             per-epoch losses it prints beside the golden model's, and
                                             check_post_training_output().

The network is the Deployer's own default example (TrainLib_Deployer.py, NET = 0): conv2d 3x3 stride 2 with bias, ReLU,
three depthwise + pointwise pairs with ReLU / Sigmoid / LeakyReLU between them, Linear 512 -> 2 with bias; MSE loss,
SGD (lr 0.01), every layer updated, 3 epochs, all tensors "in L1" (no DMA staging).  The copy of the library the Deployer
drops into the project (lib/) is deleted: the project is built against include/ of this repository or against the
reference checkout, never against a copy.
"""
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "deployer")
NAME = "Test_CNN"

DRIVER = r'''
import sys
import deployer_utils.DNN_Composer as composer
out, name = sys.argv[1], sys.argv[2]
n = 12
layers = ['conv2d', 'ReLU', 'DW', 'PW', 'ReLU', 'DW', 'PW', 'Sigmoid', 'DW', 'PW', 'LeakyReLU', 'linear']
cin = [3, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8 * 8 * 8]
cout = [8] * 11 + [2]
hk = [3, 1, 3, 1, 1, 3, 1, 1, 5, 1, 1, 1]
hin = [32, 16, 16, 14, 14, 14, 12, 12, 12, 8, 8, 1]
stride = [2] + [1] * 11
pad = [1] + [0] * 11
zeros = [0] * n
sumnodes = composer.AdjustResConnList([0] * n)
update = [1] * n
composer.CheckResConn(layers, cin, cout, hin, hin, sumnodes, update)
composer.DNN_Composer(out + '/' + name + '/', name, layers, cin, cout, hk, list(hk), hin, list(hin), stride, list(stride), pad, list(pad),
                      3, 1, 0.01, 0.1, "SGD", "MSELoss", 8, ['FP32'] * n, [1] + [0] * 10 + [1], update, zeros, zeros, zeros,
                      sumnodes, 'NO', False, True, False, True)
'''


def project_dir():
    return os.path.join(OUT, NAME)


def cflags(proj):
    """the -D flags the project's own Makefile passes (matmul selectors per layer, cluster build switches)"""
    mk = open(os.path.join(proj, "Makefile")).read()
    flags = ["-D%s=%s" % (m.group(1), m.group(2)) for m in re.finditer(r"^(MATMUL_TYPE_[A-Z]+_L\d+)\?=(\d+)", mk, flags=re.M)]
    return flags + ["-DCLUSTER", "-DFABRIC", "-DPROF_NET", "-DSTATS"]


def build_against(proj, exe, include_dirs, lib_dir, lib, num_cores, extra=()):
    cmd = ["gcc", "-O2", "-w", "-DNUM_CORES=%d" % num_cores] + cflags(proj) + list(extra) + ["-I" + proj] + ["-I" + d for d in include_dirs]
    cmd += [os.path.join(proj, "main.c"), os.path.join(proj, "net.c"), "-L" + lib_dir, "-l" + lib, "-Wl,-rpath," + lib_dir, "-lm", "-o", exe]
    subprocess.check_call(cmd)
    return exe


def build_b200(proj, exe):
    """the unmodified project against this repository's headers and libtrainlib_b200.so"""
    return build_against(proj, exe, [os.path.join(ROOT, "include")], os.path.join(ROOT, "pulp-trainlib_b200"), "trainlib_b200", 8)


def parse_run(text):
    """numbers a run prints: outputs of the last layer before and after training, the loss of every epoch, and the bit
    patterns of the final output where the project prints them"""
    out = {"loss": [float(m) for m in re.findall(r"train_loss = ([-+0-9.eE]+|nan|inf)", text)],
           "gm_loss": [float(m) for m in re.findall(r"\(GM: ([-+0-9.eE]+|nan|inf)\)", text)],
           "ideal_hex": [int(h, 16) for h in re.findall(r"Ideal = [-+0-9.eE]+ \[HEX: 0x([0-9a-fA-F]+)\]", text)],
           "mismatch": "NOT MATCHING GOLDEN MODEL" in text,
           "hex": [int(h, 16) for h in re.findall(r"Actual = [-+0-9.eE]+ \[HEX: 0x([0-9a-fA-F]+)\]", text)],
           "outputs": []}
    for block in re.findall(r"Layer \d+ output:\s*\n((?:[-+0-9.eE]+ *\n)+)", text):
        out["outputs"].append([float(v) for v in block.split()])
    return out


def generate(ref):
    deployer = os.path.join(ref, "tools", "TrainLib_Deployer")
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    os.makedirs(OUT)
    # the Deployer copies its source files by paths relative to its own directory
    subprocess.check_call([sys.executable, "-c", DRIVER, OUT, NAME], cwd=deployer, stdout=subprocess.DEVNULL)
    proj = project_dir()
    shutil.rmtree(os.path.join(proj, "lib"), ignore_errors=True)
    subprocess.check_call([sys.executable, os.path.join("utils", "GM.py")], cwd=proj, stdout=subprocess.DEVNULL)
    for f in os.listdir(proj):                      # the Deployer copies read-only files
        os.chmod(os.path.join(proj, f), 0o755 if os.path.isdir(os.path.join(proj, f)) else 0o644)
    shim = os.path.join(HERE, "shim")
    exe = build_against(proj, os.path.join(proj, "net_ref"), [shim, os.path.join(ref, "lib", "include")], os.path.join(HERE, "_ref"), "pulp_ref", 1,
                        extra=["-include", os.path.join(shim, "pmsis.h")])
    text = subprocess.check_output([exe], timeout=600).decode()
    open(os.path.join(proj, "reference_run.txt"), "w").write(text)
    os.remove(exe)
    return proj


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRAINLIB_REF", os.path.join(ROOT, "..", "reference"))
    p = generate(ref)
    print("wrote", p, parse_run(open(os.path.join(p, "reference_run.txt")).read()))
