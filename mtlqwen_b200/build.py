"""Builds libinfeng.so (CUDA kernels + C-ABI device layer + host engine) in-tree for sm_100a.

The reference compiles its engine on first import with `xcrun clang++` (runtime/inference.py:11-24);
here the same happens with nvcc, and the shared library lands beside the package so it is found
without any install step.
"""
import fcntl
import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIB = PACKAGE / "lib" / "libinfeng.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-pthread", "--expt-relaxed-constexpr"]


def sources():
  return sorted([*CSRC.glob("*.cu"), *CSRC.glob("*.cpp")])


def stale():
  if not LIB.exists():
    return True
  built = LIB.stat().st_mtime
  inputs = [*sources(), *CSRC.glob("*.h"), *CSRC.glob("*.hpp"), *CSRC.glob("*.cuh"), *(PACKAGE.parent / "include").glob("*.h")]
  return any(path.stat().st_mtime > built for path in inputs)


def build(force=False, verbose=False):
  """Compiles every source under csrc/ and links the shared library. Returns its path.
  INFENG_LIBRARY names a prebuilt library to load instead (nothing is compiled then)."""
  prebuilt = os.environ.get("INFENG_LIBRARY")
  if prebuilt and not force:
    return Path(prebuilt)
  if not force and not stale():
    return LIB
  # Several ranks of one launch may find the library stale at the same moment: one builds, the others wait and then
  # find it fresh. The link goes to a temporary name and is moved into place, so nobody loads a half-written file.
  LIB.parent.mkdir(parents=True, exist_ok=True)
  with open(LIB.parent / ".build.lock", "w") as lock:
    fcntl.flock(lock, fcntl.LOCK_EX)
    if not force and not stale():
      return LIB
    return _compile_and_link(force, verbose)


def _compile_and_link(force, verbose):
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not Path(nvcc).exists():
    raise RuntimeError("nvcc not found: libinfeng.so cannot be built")
  objects = PACKAGE / "lib" / "obj"
  objects.mkdir(parents=True, exist_ok=True)
  jobs = []
  for source in sources():
    target = objects / (source.stem + ".o")
    if force or not target.exists() or target.stat().st_mtime < max(p.stat().st_mtime for p in [source, *CSRC.glob("*.h"), *CSRC.glob("*.hpp"),
                                                                                               *CSRC.glob("*.cuh"),
                                                                                               *(PACKAGE.parent / "include").glob("*.h")]):
      command = [nvcc, *ARCH, *FLAGS, "-I", str(PACKAGE.parent / "include"), "-x", "cu", "-c", str(source), "-o", str(target)]
      if verbose:
        command.insert(1, "-Xptxas=-v")
      jobs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
  for source, job in jobs:
    output, _ = job.communicate()
    if verbose and output:
      print(output)
    if job.returncode:
      raise RuntimeError(f"nvcc failed on {source.name}:\n{output}")
  temporary = LIB.with_name(f".{LIB.name}.{os.getpid()}")
  link = [nvcc, *ARCH, "-shared", "-o", str(temporary), *[str(objects / (s.stem + ".o")) for s in sources()], "-Xcompiler", "-pthread"]
  result = subprocess.run(link, capture_output=True, text=True)
  if result.returncode:
    raise RuntimeError("link failed:\n" + result.stdout + result.stderr)
  os.replace(temporary, LIB)
  return LIB


if __name__ == "__main__":
  print(build(force="FORCE" in os.environ, verbose=True))
