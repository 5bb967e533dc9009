"""Writes tests/golden/engine_abi_layout.json: every struct of the reference's include/engine_api.h with its fields'
offsets and sizes, as a C compiler lays them out on x86-64. The header is read where it lies in the reference's tree
(it is not copied): its struct bodies are parsed for the field names, a small C program that includes the header prints
offsetof and sizeof for each, and the result is the table the reference's own engine_abi_layout returns
(include/engine_api.h:414-421: one row per field, "struct.field", then one row per struct).

    python tests/golden/make_engine_abi_golden.py <the reference's checkout>
"""
import json
import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    header = os.path.join(ref_root, "include", "engine_api.h")
    text = re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)
    structs = []
    for body, name in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            # "type a, b" or "type name[N]" or "const type *name"
            for part in decl.split(","):
                m = re.search(r"(\w+)\s*(\[[^\]]*\])*\s*$", part.strip())
                fields.append(m.group(1))
        structs.append((name, fields))
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{header}"', "int main(void) {", '  printf("[");']
    first = True
    for name, fields in structs:
        for f in fields:
            lines.append(f'  printf("%s[\\"{name}.{f}\\", %zu, %zu]", {"\"\"" if first else "\", \""}, offsetof({name}, {f}), sizeof((({name} *)0)->{f}));')
            first = False
    for name, _ in structs:
        lines.append(f'  printf(", [\\"{name}\\", 0, %zu]", sizeof({name}));')
    lines += ['  printf("]\\n");', "  return 0;", "}"]
    with tempfile.TemporaryDirectory() as d:
        src, exe = os.path.join(d, "layout.c"), os.path.join(d, "layout")
        open(src, "w").write("\n".join(lines))
        subprocess.run(["gcc", "-o", exe, src], check=True)
        rows = json.loads(subprocess.run([exe], check=True, capture_output=True, text=True).stdout)
    out = os.path.join(HERE, "engine_abi_layout.json")
    json.dump(dict(source="include/engine_api.h of avra-m3/c0ven, ENGINE_API_VERSION 23; x86-64, gcc", rows=rows), open(out, "w"), indent=0)
    print(f"{out}: {len(rows)} rows, {len(structs)} structs")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_engine_abi_golden.py <the reference's checkout>")
    main(sys.argv[1])
