"""Kernel instantiations the GPU tests need: (kind, configuration text, fp16-table mask) tuples for
quick-mlp_b200/prebuild.py. The build step runs this list ahead of time (nvcc cross-compiles without a GPU), so that
the test run on the GPU box finds every instantiation in the cache and spends no time compiling."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(HERE, "..", "quick-mlp_b200"), os.path.join(HERE, "..", "oracle"), HERE):
    if _p not in sys.path:
        sys.path.insert(0, _p)


def jobs():
    import specs
    import test_gpu_network as tn
    import test_gpu_encoding_activation as te
    import test_gpu_trainer as tt
    out = []
    for name, (cfg, _, _) in tn.network_cases().items():
        out.append(("net", json.dumps(cfg), 0))
    for name, mask in (("config3_small", 1), ("config4_small", 3), ("config5_small", 1), ("grid2d_add_plus_identity", 1)):
        out.append(("net", json.dumps(tn.network_cases()[name][0]), mask))   # fp16 table variants
    for cfg in (tt.smooth_config3(), specs.config3(log2_hashmap_size=14)):
        out.append(("net", json.dumps(cfg), 0))
        out.append(("net", json.dumps(cfg), 1))
    out.append(("net", json.dumps(tt.two_grid_config()), 3))
    for d in (2, 4):
        out.append(("net", json.dumps(tt.dims_config(d)), 0))
    import test_gpu_full_size as tf
    for cfg, mask in tf.bounds_check_jobs():
        out.append(("net", json.dumps(cfg), mask, "bounds"))
    for cfg in tf.probe_encodings():
        out.append(("enc", json.dumps(cfg), 0))
    for name, cfg in te.encoding_cases().items():
        out.append(("enc", json.dumps(cfg), 0))
    for cfg in (specs.hashgrid(3, 6, 1, 14, 8, 300), specs.hashgrid(4, 4, 1, 16, 8, 64), specs.hashgrid(2, 5, 1, -1, 4, 64)):
        out.append(("enc", json.dumps(cfg), 0))
    for a in ("relu", "celu", "sine", "identity", json.dumps(tn.LEAKY)):
        out.append(("act", a, 0))
    return out
