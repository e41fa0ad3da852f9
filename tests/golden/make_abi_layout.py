"""Writes tests/golden/abi_layout.json: sizeof/offsetof of every hot-path argument struct as the
REFERENCE's own headers (lib/include/*.h) lay them out on x86-64.  Needs the reference checkout:

    python tests/golden/make_abi_layout.py [path of the reference checkout]
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

if __name__ == "__main__":
    from conftest import load_pkg
    import abi_layout
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TRAINLIB_REF", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))
    structs = {k: v for k, v in load_pkg().abi.STRUCT_FIELDS.items()}
    layout = abi_layout.reference(structs, ref)
    json.dump(layout, open(os.path.join(HERE, "abi_layout.json"), "w"), indent=0, sort_keys=True)
    print("wrote %d structs" % len(layout))
