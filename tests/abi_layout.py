"""sizeof/offsetof of every struct of include/trainlib_b200_abi.h, measured by compiling a
generated C program against a chosen include directory (ours or the reference's)."""
import json
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _program(structs, include_line):
    lines = [include_line, "#include <stddef.h>", "#include <stdio.h>", "int main(void){", 'printf("{\\n");']
    first = True
    for name, fields in sorted(structs.items()):
        sep = "" if first else ","
        first = False
        lines.append('printf("%s\\"%s\\": {\\"sizeof\\": %%zu", sizeof(struct %s));' % (sep, name, name))
        for f, _ in fields:
            lines.append('printf(", \\"%s\\": %%zu", offsetof(struct %s, %s));' % (f, name, f))
        lines.append('printf("}\\n");')
    lines += ['printf("}\\n");', "return 0;}"]
    return "\n".join(lines)


def measure(structs, include_dirs, include_line, extra_flags=()):
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "layout.c"); exe = os.path.join(d, "layout")
        open(src, "w").write(_program(structs, include_line))
        cmd = ["gcc", "-std=gnu11", "-w"] + list(extra_flags) + ["-I" + i for i in include_dirs] + [src, "-o", exe]
        subprocess.check_call(cmd)
        return json.loads(subprocess.check_output([exe]).decode())


def ours(structs):
    return measure(structs, [os.path.join(ROOT, "include")], '#include "pulp_train.h"')


REF_DEFAULT = os.environ.get("TRAINLIB_REF", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))


def reference(structs, ref=REF_DEFAULT):
    shim = os.path.join(ROOT, "oracle", "shim")
    # pulp_train.h of the reference leaves out the RMS-norm headers
    return measure(structs, [shim, os.path.join(ref, "lib", "include")], '#include "pulp_train.h"\n#include "pulp_rmsnorm_fp32.h"\n#include "pulp_rmsnorm_fp16.h"',
                   extra_flags=["-include", os.path.join(shim, "pmsis.h")])
