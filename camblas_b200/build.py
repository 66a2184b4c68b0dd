"""Compile libcamblas_cuda.so for sm_100a with nvcc, in-tree.

The library is a single translation unit (``csrc/camblas_cuda.cu``) that
includes the kernel headers beside it. It links only the CUDA runtime; the one
driver entry point it needs (the tensor-map encoder) is looked up at run time.
The counterpart in the reference is ``scripts/build_cuda.py:68-91``, which
builds ``backend.cu`` for ``sm_90`` against cuBLAS and cuBLASLt.
"""

import hashlib
import json
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
SOURCES = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libcamblas_cuda.so"
RECORD = PACKAGE / "build.json"
FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--cudart=shared",
    "-Xcompiler",
    "-fPIC",
    "-shared",
    "-Xlinker",
    "-soname,libcamblas_cuda.so",
]


def source_digest():
    """Return one SHA-256 over every file the library is compiled from."""
    digest = hashlib.sha256()
    files = sorted(SOURCES.glob("*.cu*")) + [PACKAGE.parent / "include" / "camblas_cuda.h"]
    for path in files:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def build(force=False, verbose=False):
    """Build the shared library unless an up-to-date one exists.

    Parameters
    ----------
    force : bool
        Rebuild even when the recorded source digest matches.
    verbose : bool
        Pass ``-Xptxas -v`` so register and shared-memory use is printed.

    Returns
    -------
    pathlib.Path
        Path of the built library.
    """
    digest = source_digest()
    if not force and LIBRARY.is_file() and RECORD.is_file():
        try:
            if json.loads(RECORD.read_text()).get("sources") == digest:
                return LIBRARY
        except ValueError:
            pass
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    command = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []),
               str(SOURCES / "camblas_cuda.cu"), "-o", str(LIBRARY)]
    subprocess.run(command, check=True)
    RECORD.write_text(json.dumps({
        "command": command,
        "sources": digest,
        "library": hashlib.sha256(LIBRARY.read_bytes()).hexdigest(),
    }, indent=1))
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
