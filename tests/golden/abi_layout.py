"""Layout record of a set of C headers: every struct's size and member offsets, every enumerator's and macro constant's value.

Used twice: by tests/test_host_abi.py on this library's include/*.h, and (run as a script where the original
project's tree is at hand) on the original's headers of the same path, to write tests/golden/reference_abi_layout.txt:

    python tests/golden/abi_layout.py <original project>/include > tests/golden/reference_abi_layout.txt
    python tests/golden/abi_layout.py --symbols <original project>/include > tests/golden/reference_header_symbols.txt

(the second form lists every function those headers declare).

The struct, member and enumerator NAMES come from this library's headers (they are parsed here); the numbers come
from a C program compiled against whichever headers are asked for, so a name the other side lacks, a member of
another type or in another place, or a constant of another value all show as a difference.
"""
from __future__ import annotations

import re
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
OURS = ("rknpu_b200_w4a8.h", "rknpu_b200_quant.h", "rknpu_b200_moe.h", "rknpu_b200_rmsnorm.h")
# the original's headers that declare the same types (include/ of the original project)
THEIRS = ("rk_npu_common.h", "rk_npu_w4a8.h", "rk_npu_w4a8_tune.h", "rk_npu_matmul_i4.h", "rk_npu_quant_matmul.h",
          "rk_npu_moe_w8.h", "rk_npu_add_rmsnorm_f16.h")


def _strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def declared_names(headers=OURS):
    """-> (structs: {name: [member, ...]}, constants: [name, ...]) as this library's headers spell them; a
    constant is an enumerator or an object-like macro with a value (include guards have none)."""
    structs, enumerators = {}, []
    for header in headers:
        text = _strip_comments((ROOT / "include" / header).read_text())
        enumerators += re.findall(r"^#define[ \t]+(RK_NPU_\w+)[ \t]+\S", text, flags=re.M)
        for body, name in re.findall(r"typedef\s+struct(?:\s+\w+)?\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
            members = []
            for statement in body.split(";"):
                statement = statement.strip()
                if not statement:
                    continue
                pointer = re.search(r"\(\s*\*\s*(\w+)\s*\)", statement)      # a function pointer member
                if pointer:
                    members.append(pointer.group(1))
                    continue
                for part in statement.split(","):
                    part = re.sub(r"\[[^\]]*\]", "", part).strip()
                    members.append(re.findall(r"\w+", part)[-1])
            structs[name] = members
        for body, _ in re.findall(r"typedef\s+enum(?:\s+\w+)?\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
            for part in body.split(","):
                part = part.strip()
                if part:
                    enumerators.append(re.match(r"\w+", part).group(0))
    return structs, enumerators


def layout(include_dir: Path, headers) -> str:
    """Compile a program against `headers` under `include_dir` that prints one line per fact; return its output."""
    structs, enumerators = declared_names()
    lines = ["#include <stdio.h>", "#include <stddef.h>"] + [f'#include "{h}"' for h in headers] + ["int main(void) {"]
    for name, members in structs.items():
        lines.append(f'  printf("sizeof {name} %zu\\n", sizeof({name}));')
        for m in members:
            lines.append(f'  printf("offsetof {name} {m} %zu %zu\\n", offsetof({name}, {m}), sizeof((({name}*)0)->{m}));')
    for e in enumerators:
        lines.append(f'  printf("value {e} %lld\\n", (long long){e});')
    lines += ["  return 0;", "}"]
    with tempfile.TemporaryDirectory() as tmp:
        src, exe = Path(tmp) / "layout.c", Path(tmp) / "layout"
        src.write_text("\n".join(lines) + "\n")
        subprocess.run(["gcc", "-std=c11", "-I", str(include_dir), str(src), "-o", str(exe)], check=True, capture_output=True, text=True)
        return subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout


def functions(include_dir: Path, headers) -> list:
    """Names of the functions `headers` declare, sorted."""
    names = set()
    for header in headers:
        names |= set(re.findall(r"\b(rk_npu_\w+)\s*\(", _strip_comments((Path(include_dir) / header).read_text())))
    return sorted(names)


if __name__ == "__main__":
    if sys.argv[1] == "--symbols":
        sys.stdout.write("\n".join(functions(Path(sys.argv[2]), THEIRS)) + "\n")
    else:
        sys.stdout.write(layout(Path(sys.argv[1]), THEIRS))
