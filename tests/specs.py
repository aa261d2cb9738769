"""Network specifications used by the parity tests and the benchmark: the five BASELINE configurations and
scaled-down relatives that the CPU oracle finishes in seconds."""
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


# ---- the five BASELINE configurations ------------------------------------------------------------------------------
def config1():   # CPU Eigen reference case: 3 -> 16 relu -> 1 relu, no bias, N = 65536
    return identity_net(3, [16, 1], ["relu", "relu"], bias=False)


def config2():   # fused inference: 3 -> 64 relu -> 64 celu -> 64 sine -> 64 relu -> 1 identity, bias, N = 2^22
    return identity_net(3, [64, 64, 64, 64, 1], ["relu", "celu", "sine", "relu", "identity"])


def config3(log2_hashmap_size=19):   # hash grid training step, N = 2^20
    return grid_net(3, [hashgrid(3, 16, 2, log2_hashmap_size, 16, 7006, per_level_scale=1.5)],
                    [64, 64, 1], ["relu", "relu", "identity"])


def config4(log2_hashmap_size=18, dense_resolution=64):   # dense + hash grid, uneven widths, N = 2^21 per GPU
    return grid_net(3, [hashgrid(3, 1, 4, -1, dense_resolution, dense_resolution),
                        hashgrid(3, 8, 4, log2_hashmap_size, 32, 4096, per_level_scale=2.0)],
                    [128, 64, 16, 4], ["sine", "celu", "relu", "identity"])


def config5(log2_hashmap_size=22):   # 4-D hash grid inference, N = 2^24
    return grid_net(4, [hashgrid(4, 16, 4, log2_hashmap_size, 16, 2489)],
                    [128, 128, 128, 4], ["relu", "relu", "relu", "identity"])


def dumps(cfg) -> str:
    return json.dumps(cfg)
