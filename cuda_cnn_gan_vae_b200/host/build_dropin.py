"""Builds the drop-in proof: the reference's own sources compiled against this package's headers.

A shadow tree is laid out in a temporary directory with the reference's directory structure, in which
cuda/{ctensor,ctensormath,ctensorconv,ctensorapplyfunc,tensor}.cu.h are links to host/cuda/ of this
package and every other file is a link to the reference tree.  The reference's headers include each
other by relative path ("../cuda/tensor.cu.h"), so inside the shadow tree they pick up this package's
tensor layer without a single changed line.  Nothing of the reference is copied; the tree is removed
after the build, and the binaries, the weight file and the CPU dump under oracle/_ref/dropin/ are build
artefacts (git-ignored) that are only (re)built where the reference tree exists.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
# where the reference tree (da-nie/CUDA-CNN-GAN-VAE) is checked out: B200CONV_REFERENCE, else a "reference" directory beside this
# repository; absent on machines that only run the prebuilt checker
REF = os.environ.get("B200CONV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
OUT = os.path.join(ROOT, "oracle", "_ref", "dropin")
OURS = ("ctensor.cu.h", "ctensormath.cu.h", "ctensorconv.cu.h", "ctensorapplyfunc.cu.h", "tensor.cu.h")
# this package's own layer classes (host/netlayer/): in the second shadow tree they stand in for the reference's headers of the
# same names, next to the reference's remaining layer classes
OWN_LAYERS = ("cnetlayerconvolution.cu.h", "cnetlayerbackconvolution.cu.h", "cnetlayerlinear.cu.h", "cnetlayerbatchnormalization.cu.h",
              "b200netlayer.cu.h", "b200convlayer.cu.h")


def _link(src, dst):
    if os.path.lexists(dst):
        os.remove(dst)
    os.symlink(src, dst)


def make_shadow(shadow, own_layers=False):
    for sub in ("cuda", "netlayer", "common", "system"):
        os.makedirs(os.path.join(shadow, sub), exist_ok=True)
        for name in os.listdir(os.path.join(REF, sub)):
            src = os.path.join(REF, sub, name)
            if os.path.isfile(src) and not (sub == "cuda" and name in OURS):
                _link(src, os.path.join(shadow, sub, name))
    for name in OURS:
        _link(os.path.join(HERE, "cuda", name), os.path.join(shadow, "cuda", name))
    _link(os.path.join(REF, "settings.h"), os.path.join(shadow, "settings.h"))
    if own_layers:
        for name in OWN_LAYERS:
            _link(os.path.join(HERE, "netlayer", name), os.path.join(shadow, "netlayer", name))


def build(force=False):
    """Returns the list of built binaries, or the existing ones when the reference tree is absent."""
    targets = {"dropin_kat": "dropin_kat.cpp", "dropin_layers": "dropin_layers.cpp", "dropin_fastlayers": "dropin_fastlayers.cpp"}
    bins = {k: os.path.join(OUT, k) for k in targets}
    if not os.path.isdir(os.path.join(REF, "cuda")):
        return [b for b in bins.values() if os.path.exists(b)]
    os.makedirs(OUT, exist_ok=True)
    shadow = tempfile.mkdtemp(prefix="b200_dropin_")
    shadow_own = tempfile.mkdtemp(prefix="b200_dropin_own_")
    try:
        make_shadow(shadow_own, own_layers=True)
        return _build(force, targets, bins, shadow, shadow_own)
    finally:
        shutil.rmtree(shadow, ignore_errors=True)
        shutil.rmtree(shadow_own, ignore_errors=True)


def _build(force, targets, bins, shadow, shadow_own):
    make_shadow(shadow)
    libdir = os.path.join(ROOT, "cuda_cnn_gan_vae_b200")
    link = [os.path.join(REF, "system", "system.cpp"), os.path.join(REF, "common", "idatastream.cpp"),
            os.path.join(REF, "common", "cdatastreamfile.cpp"), os.path.join(REF, "common", "crandom.cpp")]
    built = []
    for name, src in targets.items():
        path = os.path.join(HERE, "programs", src)
        if not os.path.exists(path):
            continue
        deps = [path] + [os.path.join(HERE, "cuda", n) for n in OURS] + [os.path.join(HERE, "netlayer", n) for n in OWN_LAYERS]
        tree = shadow_own if name == "dropin_fastlayers" else shadow
        if not force and os.path.exists(bins[name]) and all(os.path.getmtime(d) <= os.path.getmtime(bins[name]) for d in deps):
            built.append(bins[name])
            continue
        cmd = ["g++", "-O2", "-std=c++14", "-w", "-I" + tree, "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
               "-o", bins[name], path] + link + ["-L" + libdir, "-lb200conv", "-L/usr/local/cuda/lib64", "-lcudart",
                                                "-Wl,-rpath,$ORIGIN/../../../cuda_cnn_gan_vae_b200", "-Wl,-rpath,/usr/local/cuda/lib64"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("drop-in build failed: " + name)
        built.append(bins[name])
    # the layer program once more against the reference's own CPU backend, its weight file and its dump
    cpu = os.path.join(OUT, "dropin_layers_cpu")
    src = os.path.join(HERE, "programs", "dropin_layers.cpp")
    if force or not os.path.exists(cpu) or os.path.getmtime(src) > os.path.getmtime(cpu):
        r = subprocess.run(["g++", "-O2", "-std=c++14", "-w", "-DUSE_CPU", "-I" + REF, "-o", cpu, src] + link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("drop-in build failed: dropin_layers_cpu")
        subprocess.run([cpu, "gen", os.path.join(OUT, "w0.net")], check=True)
        subprocess.run([cpu, "run", os.path.join(OUT, "w0.net"), os.path.join(OUT, "dump_cpu.txt")], check=True)
    built.append(cpu)
    return built


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
