"""In-tree build of libmccl.so (host C++ with g++, device code with nvcc for sm_100a).

`python -m mccl_b200._build` compiles every file under csrc/ that is newer than its object and links
mccl_b200/lib/libmccl.so.  Objects live in build/ (ignored by git); the shared library stays inside the
package so that it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
LIB = ROOT / "mccl_b200" / "lib" / "libmccl.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

CXXFLAGS = ["-O2", "-g1", "-fPIC", "-std=c++17", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread",
            f"-I{ROOT / 'include'}", f"-I{CSRC}", f"-I{CUDA_HOME / 'include'}"]
NVCCFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
             "-Xcompiler", "-fPIC,-Wall,-Wno-unused-parameter", f"-I{ROOT / 'include'}", f"-I{CSRC}",
             "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _headers_mtime() -> float:
    newest = 0.0
    for pat in ("*.h", "*.cuh"):
        for h in list(CSRC.rglob(pat)) + list((ROOT / "include").rglob(pat)):
            newest = max(newest, h.stat().st_mtime)
    return newest


def _compile(src: Path, obj: Path, verbose: bool) -> tuple[Path, str]:
    obj.parent.mkdir(parents=True, exist_ok=True)
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCCFLAGS, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXXFLAGS, "-c", str(src), "-o", str(obj)]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{p.stdout}\n{p.stderr}")
    log = p.stderr if src.suffix == ".cu" else ""
    if src.suffix == ".cu":
        (obj.with_suffix(".ptxas.txt")).write_text(p.stderr)
    return src, log


def build(verbose: bool = False, force: bool = False) -> Path:
    if shutil.which(NVCC) is None and not Path(NVCC).exists():
        raise RuntimeError(f"nvcc not found at {NVCC}")
    srcs = sorted(list(CSRC.rglob("*.cc")) + list(CSRC.rglob("*.cu")))
    hdr = _headers_mtime()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / s.relative_to(CSRC).with_suffix(s.suffix + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr):
            jobs.append((s, o))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            for src, log in ex.map(lambda so: _compile(so[0], so[1], verbose), jobs):
                if verbose:
                    print(f"[mccl build] {src.relative_to(ROOT)}")
                    if log:
                        print(log)
    if jobs or not LIB.exists():
        LIB.parent.mkdir(parents=True, exist_ok=True)
        # Linked beside the target and renamed into place: whoever copies or loads the tree never sees half a library.
        tmp = LIB.with_name(f".{LIB.name}.{os.getpid()}.tmp")
        cmd = [NVCC, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static",
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{p.stdout}\n{p.stderr}")
        os.replace(tmp, LIB)
        if verbose:
            print(f"[mccl build] linked {LIB.relative_to(ROOT)}")
    return LIB


def resources() -> str:
    """Markdown table of what ptxas reported for every kernel of the last build (registers, spills, static shared
    memory), template instantiations of one kernel folded into one row."""
    import re
    from collections import OrderedDict
    found = []
    for f in sorted(OBJ.rglob("*.ptxas.txt")):
        entry, spill = None, ("0", "0", "0")
        for line in f.read_text().splitlines():
            m = re.search(r"Compiling entry function '(\S+)' for 'sm_100a'", line)
            if m:
                entry, spill = m.group(1), ("0", "0", "0")
                continue
            m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m and entry:
                spill = m.groups()
            m = re.search(r"Used (\d+) registers", line)
            if m and entry:
                smem = re.search(r"(\d+) bytes smem", line)
                found.append((f.name.replace(".ptxas.txt", ""), entry, int(m.group(1)),
                              int(spill[1]) + int(spill[2]), int(smem.group(1)) if smem else 0))
                entry = None
    names = subprocess.run(["c++filt"], input="\n".join(k[1] for k in found), capture_output=True,
                           text=True).stdout.splitlines()
    rows: "OrderedDict[tuple, list]" = OrderedDict()
    for k, name in zip(found, names):
        name = name.replace("(anonymous namespace)::", "").replace("mccl::", "")
        name = re.sub(r"^void ", "", re.sub(r"\(.*\)$", "", name))
        base = name.split("<")[0]
        rows.setdefault((k[0], base), []).append(k)
    out = ["| file | kernel | instantiations | registers | spill bytes (stores + loads), worst | static smem bytes, worst |",
           "|---|---|---|---|---|---|"]
    for (src, base), ks in rows.items():
        regs = [k[2] for k in ks]
        out.append(f"| {src} | `{base}` | {len(ks)} | {min(regs)}" + (f" - {max(regs)}" if max(regs) != min(regs) else "")
                   + f" | {max(k[3] for k in ks)} | {max(k[4] for k in ks)} |")
    out.append("")
    out.append(f"{len(found)} kernels in {len(rows)} families; {sum(1 for k in found if k[3])} with spills.")
    return "\n".join(out)


if __name__ == "__main__":
    if "--resources" in sys.argv:
        print(resources())
    else:
        build(verbose=True, force="--force" in sys.argv)
