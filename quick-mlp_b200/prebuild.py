"""Instantiates kernel templates for a list of specs ahead of time, several nvcc processes at once.
The library would build a missing instantiation on first use; doing it here keeps compile time out of the GPU run.

Jobs are tuples ("net", cfg_json, grid_half_mask) | ("enc", cfg_json, half_table) | ("act", key_or_json, 0); a fourth
element "bounds" asks for the bounds-checking instantiation.
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def run_jobs(jobs):
    if HERE not in sys.path:
        sys.path.insert(0, HERE)
    from qmlp import bindings
    bindings.QuickMLP.set_log_level("error")
    errors = []
    for job in jobs:
        try:
            kind = job[0]
            bindings.QuickMLP.set_tuning("bounds_check", 1 if (len(job) > 3 and job[3] == "bounds") else 0)
            if kind == "net":
                bindings.Network(job[1]).compile(int(job[2]))
            elif kind == "enc":
                bindings.Encoding(job[1]).compile(bool(job[2]))
            elif kind == "act":
                bindings.Activation(job[1]).compile()
            else:
                raise ValueError(kind)
        except Exception as e:
            errors.append(f"{job[0]} {job[1][:120]}: {e}")
    return errors


def purge_stale(cache_dir=None):
    """Instantiations are named by a hash of their source and of every template header, so a header change leaves the
    old shared objects behind as dead weight. They are removed here whenever the headers differ from the ones the cache
    was last filled with."""
    import hashlib
    cache_dir = cache_dir or os.path.join(HERE, "lib", "specs")
    kernels = os.path.join(HERE, "csrc", "kernels")
    h = hashlib.sha256()
    for name in sorted(os.listdir(kernels)):
        h.update(name.encode())
        with open(os.path.join(kernels, name), "rb") as f:
            h.update(f.read())
    digest = h.hexdigest()
    stamp = os.path.join(cache_dir, "headers.stamp")
    if os.path.isdir(cache_dir):
        old = open(stamp).read() if os.path.exists(stamp) else ""
        if old != digest:
            for name in os.listdir(cache_dir):
                if name.startswith("qmlp_") and name.rsplit(".", 1)[-1] in ("so", "cu", "log"):
                    os.unlink(os.path.join(cache_dir, name))
    os.makedirs(cache_dir, exist_ok=True)
    with open(stamp, "w") as f:
        f.write(digest)


def prebuild(jobs, processes=None):
    jobs = [list(j) for j in dict.fromkeys(tuple(j) for j in jobs)]
    if not jobs:
        return
    purge_stale()
    processes = max(1, min(len(jobs), processes or os.cpu_count() or 4))
    with tempfile.TemporaryDirectory() as tmp:
        procs = []
        for i in range(processes):
            path = os.path.join(tmp, f"jobs{i}.json")
            with open(path, "w") as f:
                json.dump(jobs[i::processes], f)
            procs.append(subprocess.Popen([sys.executable, os.path.abspath(__file__), path],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        failed = []
        for p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                failed.append(out[-4000:])
    if failed:
        raise RuntimeError("kernel instantiation failed:\n" + "\n".join(failed))


if __name__ == "__main__":
    with open(sys.argv[1]) as f:
        errs = run_jobs(json.load(f))
    if errs:
        print("\n".join(errs))
        sys.exit(1)
