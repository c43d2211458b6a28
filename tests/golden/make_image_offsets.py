"""Writes tests/golden/image_header_offsets.json: byte offset and size of every
field of the reference's layer-image headers, as the reference's own header
files lay them out.  Needs the reference tree and gcc; run from the repository
root:

    python tests/golden/make_image_offsets.py /path/to/reference

The JSON pins the restated layouts in the library (csrc/q4b_image.cu) and in the
image writer (cpu-llms-in-c_b200/image.py)."""
import json
import os
import re
import subprocess
import sys
import tempfile

HEADERS = {
    "delta": ("qwen38_m3_image.h", "qwen38_m3_image_header"),
    "attention": ("qwen38_m3_attention_image.h", "qwen38_m3_attention_image_header"),
    "global": ("qwen38_m3_global_image.h", "qwen38_m3_global_image_header"),
    "mtp": ("qwen38_m3_mtp_image.h", "qwen38_m3_mtp_image_header"),
}


def fields_of(text: str, struct: str) -> list[str]:
    body = text[:text.index("} " + struct)]
    body = body[body.rindex("typedef struct {") + len("typedef struct {"):]
    names = []
    for line in body.split(";"):
        match = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*(\[[^;]*\])?\s*$", line.strip(), re.S)
        if match:
            names.append(match.group(1))
    return names


def main(reference_root: str) -> None:
    include = os.path.join(reference_root, "models", "qwen3.8-27b", "targets", "apple-m3-pro")
    result = {}
    for key, (header, struct) in HEADERS.items():
        with open(os.path.join(include, header)) as handle:
            names = fields_of(handle.read(), struct)
        lines = [f'#include <stdio.h>\n#include <stddef.h>\n#include "{header}"\nint main(void) {{']
        for name in names:
            lines.append(f'printf("%s %zu %zu\\n", "{name}", offsetof({struct}, {name}), sizeof((({struct} *)0)->{name}));')
        lines.append(f'printf("sizeof %zu 0\\n", sizeof({struct})); return 0; }}')
        with tempfile.TemporaryDirectory() as scratch:
            source = os.path.join(scratch, "offsets.c")
            with open(source, "w") as handle:
                handle.write("\n".join(lines))
            binary = os.path.join(scratch, "offsets")
            subprocess.check_call(["gcc", "-std=c11", "-I", include, source, "-o", binary])
            output = subprocess.check_output([binary]).decode()
        result[key] = {name: [int(offset), int(size)] for name, offset, size in
                       (line.split() for line in output.strip().splitlines())}
    target = os.path.join(os.path.dirname(os.path.abspath(__file__)), "image_header_offsets.json")
    with open(target, "w") as handle:
        json.dump(result, handle, indent=1)
    print("wrote", target)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE", "")
    if not root:
        raise SystemExit("usage: make_image_offsets.py <reference checkout>   (or REFERENCE in the environment)")
    main(root)
