"""Build recipe for the CPU oracle (test infrastructure, never part of the product library).

  oracle/liboracle.so      plain-C restatement (oracle/oracle.c); always built.
  oracle/_ref/libref.so    the reference's own CPU backend, compiled in place from the reference
                           tree (nothing is copied) behind the C-ABI of oracle/ref_shim.cpp.
  oracle/_ref/ref_selftest the reference's own known-answer suite on its CPU backend.

The two _ref artefacts are only (re)built when the reference tree is present; a machine without
it uses the prebuilt files that travelled with the repository snapshot.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference tree (da-nie/CUDA-CNN-GAN-VAE) is checked out: B200CONV_REFERENCE, else a "reference" directory beside this
# repository; absent on machines that only run the prebuilt checker
REF = os.environ.get("B200CONV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_DIR = os.path.join(HERE, "_ref")


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed: " + cmd[0])


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    src = os.path.join(HERE, "oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if force or _stale(out, [src]):
        _run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-o", out, src, "-lm"])
    return out


def build_ref(force=False):
    """Compile the reference CPU backend when its tree is present; return the .so path or None."""
    out = os.path.join(REF_DIR, "libref.so")
    selftest = os.path.join(REF_DIR, "ref_selftest")
    if not os.path.isdir(os.path.join(REF, "cpu")):
        return out if os.path.exists(out) else None
    os.makedirs(REF_DIR, exist_ok=True)
    link = [os.path.join(REF, "system", "system.cpp"),
            os.path.join(REF, "common", "idatastream.cpp"),
            os.path.join(REF, "common", "cdatastreamfile.cpp")]
    flags = ["-O3", "-std=c++14", "-fPIC", "-w", "-ffp-contract=off", "-I" + REF, "-I" + os.path.join(REF, "cpu")]
    shim = os.path.join(HERE, "ref_shim.cpp")
    if force or _stale(out, [shim]):
        # -DUSE_CPU: the reference's layer headers (the VAE output layer) then include its CPU tensor backend
        _run(["g++"] + flags + ["-DUSE_CPU", "-shared", "-o", out, shim, os.path.join(REF, "common", "crandom.cpp")] + link)
    st = os.path.join(HERE, "ref_selftest.cpp")
    if force or _stale(selftest, [st]):
        _run(["g++"] + flags + ["-DUSE_CPU", "-I" + os.path.join(REF, "cuda"), "-o", selftest, st,
                                os.path.join(REF, "common", "crandom.cpp")] + link)
    return out


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
