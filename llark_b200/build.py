"""Builds the CUDA library on demand. `make` builds libllark_b200.so (everything); `make serve` builds
libllark_serve.so: the GEMM core, the decode linears and the generation-path ops of the layer-list decoders, which is
all a native checkpoint needs. `ensure_built()` is what the command-line tools call first: it does nothing when a
library is there, otherwise it compiles the serve subset (a lock file keeps two first calls from racing)."""
import fcntl
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "llark_b200")
FULL = os.path.join(PKG, "libllark_b200.so")
SERVE = os.path.join(PKG, "libllark_serve.so")


def _sources_newer_than(lib, names):
    t = os.path.getmtime(lib)
    paths = [os.path.join(PKG, "csrc", n) for n in names] + [os.path.join(ROOT, "include", "llark_b200.h")]
    return any(os.path.exists(p) and os.path.getmtime(p) > t for p in paths)


SERVE_SOURCES = ("gemm_tcgen05.cu", "gemv.cu", "seq_ops.cu", "seq_mixers.cu", "seq_swa_mma.cu", "seq_delta.cu",
                 "seq_latent.cu", "seq_moe.cu", "common.cuh")


def ensure_built(verbose=False):
    """Path of a usable library; compiles the serve subset if there is none (or its sources are newer)."""
    if os.environ.get("LLARK_LIB_PATH"):
        return os.environ["LLARK_LIB_PATH"]
    for lib in (FULL, SERVE):
        if os.path.exists(lib) and not _sources_newer_than(lib, SERVE_SOURCES):
            return lib
    os.makedirs(os.path.join(ROOT, "build"), exist_ok=True)
    with open(os.path.join(ROOT, "build", ".serve.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if os.path.exists(SERVE) and not _sources_newer_than(SERVE, SERVE_SOURCES):
            return SERVE
        env = dict(os.environ)
        env["PATH"] = "/usr/local/cuda/bin:" + env.get("PATH", "")
        r = subprocess.run(["make", "-j8", "-C", ROOT, "serve"], env=env, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout[-4000:] + r.stderr[-4000:])
        if r.returncode != 0:
            raise RuntimeError("building libllark_serve.so failed")
    return SERVE


if __name__ == "__main__":
    print(ensure_built(verbose=True))
