"""Static checks over the source tree: declared environment knobs, forbidden identifiers, source-only history."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_EXT = (".py", ".cu", ".cuh", ".h", ".cpp")


def _sources():
    for top in ("vllm_torchtpu_b200", "tests", "benchmarks", "examples"):
        for d, _, files in os.walk(os.path.join(ROOT, top)):
            if "__pycache__" in d or os.sep + "build" in d:
                continue
            for f in files:
                if f.endswith(SRC_EXT):
                    yield os.path.join(d, f)
    for f in ("bench.py", "__graft_entry__.py"):
        yield os.path.join(ROOT, f)


def test_every_environment_knob_that_is_read_is_declared():
    from vllm_torchtpu_b200 import envs
    declared = set(envs.declared())
    used = set()
    for p in _sources():
        if p.endswith(".py") and os.sep + "tests" + os.sep not in p:
            used |= set(re.findall(r"\benvs\.(B200_[A-Z0-9_]+)", open(p).read()))
    assert used <= declared, sorted(used - declared)
    # knobs the kernel library reads with getenv are declared as well
    c_side = set()
    for p in _sources():
        if p.endswith((".cu", ".cpp", ".h", ".cuh")):
            c_side |= set(re.findall(r'getenv\("(B200_[A-Z0-9_]+)"\)', open(p).read()))
    assert c_side <= declared, sorted(c_side - declared)


def test_sources_do_not_name_closed_calls_or_cluster_multicast_loads():
    this = os.path.abspath(__file__)
    batched = re.compile("cu(da)?Memcpy(3D)?" + "Batch" + "Async")
    multicast = re.compile(r"cp\.async\.bulk[^\n;]*\.multicast" + "::cluster")
    for p in _sources():
        if os.path.abspath(p) == this:
            continue
        text = open(p, errors="ignore").read()
        assert not batched.search(text), p
        assert not multicast.search(text), p


def test_built_artifacts_are_not_tracked():
    import subprocess
    r = subprocess.run(["git", "ls-files"], cwd=ROOT, capture_output=True, text=True)
    if r.returncode != 0:
        return                      # not a git checkout (e.g. a copied tree)
    tracked = r.stdout.split("\n")
    assert not [f for f in tracked if f.endswith((".so", ".o", ".ncu-rep")) or f.startswith(("_work/", "gpurun_out/"))]
