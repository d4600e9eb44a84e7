#!/usr/bin/env python3
"""Writes the compile-time CUDA hook into a copy of the reference's nntrainer/tensor/float_tensor.cpp.

The reference dispatches a block-quantized weight product in FloatTensor::dotQnK (float_tensor.cpp:923-969) to
gemm_q4_K / gemm_q6_K / gemm_q4_0 of cpu_backend.h, and already has one compile-time branch there for another device
backend (#ifdef ENABLE_OPENCL, float_tensor.cpp:953-961). This tool adds the same kind of branch for this library: every
such call inside dotQnK becomes

    #ifdef ENABLE_CUDA
        gemm_q4_K_cuda(<the same arguments>);
    #else
        gemm_q4_K(<the same arguments>);
    #endif

and `#include <cuda_backend.h>` is added under the same macro. Nothing else of the file changes, and a build without
-DENABLE_CUDA compiles exactly what it compiled before.

    python plugin/hook_dotqnk.py <reference>/nntrainer/tensor/float_tensor.cpp > float_tensor.cpp

The function is found by name and its body by brace matching, so the tool does not depend on line numbers.
"""
from __future__ import annotations

import re
import sys

CALL = re.compile(r"^(?P<indent>[ \t]*)(?P<fn>gemm_q4_K|gemm_q6_K|gemm_q4_0)\((?P<args>[^;]*)\);[ \t]*$")
INCLUDE = "#ifdef ENABLE_CUDA\n#include <cuda_backend.h>\n#endif\n"


def body_span(lines: list[str], start: int) -> tuple[int, int]:
    """Lines [first, last] of the brace-matched body that opens at or after line ``start``."""
    depth, first = 0, None
    for i in range(start, len(lines)):
        for ch in lines[i]:
            if ch == "{":
                depth += 1
                if first is None:
                    first = i
            elif ch == "}":
                depth -= 1
                if first is not None and depth == 0:
                    return first, i
    raise ValueError("unbalanced braces after FloatTensor::dotQnK")


def hook(source: str) -> tuple[str, int]:
    """Returns the hooked text and the number of calls that were wrapped."""
    if "ENABLE_CUDA" in source:
        raise ValueError("the file already mentions ENABLE_CUDA")
    lines = source.splitlines(keepends=True)
    heads = [i for i, ln in enumerate(lines) if "FloatTensor::dotQnK(" in ln]
    if len(heads) != 1:
        raise ValueError(f"expected one definition of FloatTensor::dotQnK, found {len(heads)}")
    first, last = body_span(lines, heads[0])
    out, wrapped = [], 0
    for i, ln in enumerate(lines):
        m = CALL.match(ln.rstrip("\n")) if first <= i <= last else None
        if m is None:
            out.append(ln)
            continue
        ind, fn, args = m.group("indent"), m.group("fn"), m.group("args")
        out.append(f"#ifdef ENABLE_CUDA\n{ind}{fn}_cuda({args});\n#else\n{ln if ln.endswith(chr(10)) else ln + chr(10)}#endif\n")
        wrapped += 1
    if wrapped == 0:
        raise ValueError("no gemm_q4_K / gemm_q6_K / gemm_q4_0 call found inside FloatTensor::dotQnK")
    # the include goes right behind the header whose functions the hook stands in for (a later #include of the file may
    # sit inside another backend's conditional block)
    text = "".join(out)
    m = re.search(r"^#include <cpu_backend\.h>[^\n]*\n", text, flags=re.M)
    if m is None:
        raise ValueError("the file does not include <cpu_backend.h>")
    return text[:m.end()] + INCLUDE + text[m.end():], wrapped


def main(argv: list[str]) -> int:
    if len(argv) != 2:
        sys.stderr.write(__doc__)
        return 2
    with open(argv[1], encoding="utf-8") as f:
        text, n = hook(f.read())
    sys.stdout.write(text)
    sys.stderr.write(f"hook_dotqnk: {n} calls wrapped\n")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
