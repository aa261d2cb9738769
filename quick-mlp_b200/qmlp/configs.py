"""Network specifications of the five benchmark configurations (JSON spec format of the reference,
src_cpp/src/fused_network.cpp:33-139, README.md:68-110) and small builders for relatives of them.

The benchmark, the build step and the parity tests all take their specs from here, so that the network a number is
quoted on is the network the tests check.
"""
import json

BUILTIN = ["qmlp/builtin-activations.json"]


def mlp(widths, activations, bias=True):
    return [{"n_out": w, "bias": bias if isinstance(bias, bool) else bias[i], "activation": a}
            for i, (w, a) in enumerate(zip(widths, activations))]


def identity_net(n_in, widths, activations, bias=True, extra_activations=()):
    return {"num_inputs": n_in, "num_outputs": widths[-1],
            "activation_specification": BUILTIN + list(extra_activations),
            "encodings": [{"id": "Identity", "start_in": 0, "n_in": n_in}],
            "network": mlp(widths, activations, bias)}


def hashgrid(n_in, n_levels, n_features, log2_hashmap_size, min_resolution, max_resolution, per_level_scale=None,
             combination_mode="concat", start_in=0, box_min=None, box_size=None):
    e = {"id": "HashGrid", "start_in": start_in, "n_in": n_in, "n_levels": n_levels,
         "n_features_per_level": n_features, "log2_hashmap_size": log2_hashmap_size,
         "min_resolution": min_resolution, "max_resolution": max_resolution, "combination_mode": combination_mode,
         "bounding_box_min": box_min if box_min is not None else [0.0] * n_in,
         "bounding_box_size": box_size if box_size is not None else [1.0] * n_in}
    if per_level_scale is not None:
        e["per_level_scale"] = per_level_scale
    return e


def grid_net(n_in, encodings, widths, activations, bias=True):
    return {"num_inputs": n_in, "num_outputs": widths[-1], "activation_specification": BUILTIN,
            "encodings": encodings, "network": mlp(widths, activations, bias)}


# ---- the five benchmark configurations ------------------------------------------------------------------------------
def config1():
    """Identity encoding, 3 -> 16 relu -> 1 relu, no bias (the shape of the reference's CPU comparison tests); 65536 points."""
    return identity_net(3, [16, 1], ["relu", "relu"], bias=False)


def config2():
    """Identity encoding, 3 -> 64 relu -> 64 celu -> 64 sine -> 64 relu -> 1 identity, bias; fused inference of 2^22 points."""
    return identity_net(3, [64, 64, 64, 64, 1], ["relu", "celu", "sine", "relu", "identity"])


def config3(log2_hashmap_size=19):
    """3-D hash grid (16 levels x 2 features, 2^19 rows per hashed level, resolutions 16 * 1.5^l) + 32 -> 64 relu -> 64
    relu -> 1; training step on 2^20 points."""
    return grid_net(3, [hashgrid(3, 16, 2, log2_hashmap_size, 16, 7006, per_level_scale=1.5)],
                    [64, 64, 1], ["relu", "relu", "identity"])


def config4(log2_hashmap_size=18, dense_resolution=64):
    """Dense 64^3 x 4 grid + 3-D hash grid (8 levels x 4 features, 2^18 rows, resolutions 32 * 2^l), concatenated to 36
    features -> 128 sine -> 64 celu -> 16 relu -> 4; data-parallel training on 2^21 points per GPU."""
    return grid_net(3, [hashgrid(3, 1, 4, -1, dense_resolution, dense_resolution),
                        hashgrid(3, 8, 4, log2_hashmap_size, 32, 4096, per_level_scale=2.0)],
                    [128, 64, 16, 4], ["sine", "celu", "relu", "identity"])


def config5(log2_hashmap_size=22):
    """4-D hash grid (16 levels x 4 features, 2^22 rows, resolutions 16 ... 2489) + 64 -> 128 relu x 3 -> 4; inference of
    2^24 points sharded over the GPUs."""
    return grid_net(4, [hashgrid(4, 16, 4, log2_hashmap_size, 16, 2489)],
                    [128, 128, 128, 4], ["relu", "relu", "relu", "identity"])


CONFIGS = {"c1": config1, "c2": config2, "c3": config3, "c4": config4, "c5": config5}

# Per-point algorithmic work of each workload: flops = sum over the unpadded layers of 2 * in * out (a training step
# counts forward, input-gradient and weight-gradient contractions: 3x); bytes = fp32 inputs + fp32 outputs + the fp16
# grid rows a point consumes (levels * 2^D corners * features * 2 B) and, for a training step, the fp32 gradient rows it
# adds to (read-modify-write: 2 * 4 B per element) and the stash of layer inputs written and read once.
WORKLOADS = {
    "c1": dict(points=1 << 16, mode="inference", flops=128, bytes=16, lo=0.0, hi=1.0,
               name="config1: identity 3->16 relu->1 relu, no bias, 65536 points, fused inference"),
    "c2": dict(points=1 << 22, mode="inference", flops=25088, bytes=16, lo=-1.0, hi=1.0,
               name="config2: identity 3->64 relu->64 celu->64 sine->64 relu->1, bias, 2^22 points, fused inference"),
    "c3": dict(points=1 << 20, mode="train", flops=3 * 12416, bytes=3100, gather_bytes=512, lo=0.0, hi=1.0,
               name="config3: 3-D hash grid 16x2 (2^19) + 32->64->64->1, 2^20 points, fused training step"),
    "c3i": dict(points=1 << 20, mode="inference", flops=12416, bytes=528, gather_bytes=512, lo=0.0, hi=1.0, config="c3",
                name="config3: 3-D hash grid 16x2 (2^19) + 32->64->64->1, 2^20 points, fused inference"),
    "c4": dict(points=1 << 21, mode="train", flops=3 * 27776, bytes=3600, gather_bytes=576, lo=0.0, hi=1.0,
               name="config4: dense 64^3x4 + hash 8x4 (2^18) + 36->128->64->16->4, 2^21 points per GPU, training step"),
    "c5": dict(points=1 << 24, mode="inference", flops=82944, bytes=2080, gather_bytes=2048, lo=0.0, hi=1.0, sharded=True,
               name="config5: 4-D hash grid 16x4 (2^22) + 64->128x3->4, 2^24 points sharded over the GPUs, fused inference"),
}


def workload_config(key):
    return CONFIGS[WORKLOADS[key].get("config", key)]()


def dumps(cfg) -> str:
    return json.dumps(cfg)
