"""Reading and writing the reference's model file: the YAML that training/export.py:55-99 writes and
example/load_model.hpp:25-52 reads.

    geometry: {shape: SPHERE, radius: 0.0949996, intersections: 6, ...}
    mesh: RING6
    network:                      # list of convolutional groups
      - - activation: selu        #   list of dense layers of the group
          biases: [...]           #     n_out
          weights: [[...], ...]   #     n_in rows of n_out values: [in][out], cpp/visualmesh/network_structure.hpp:25-27

The first layer's rows are (N+1) * 4: the exporter pads a 3-channel network with zero alpha rows (export.py:83-89).
"""
from typing import Tuple

import numpy as np
import yaml

from .workloads import RELU, SELU, SOFTMAX, TANH, Layer, Network

_ACTIVATIONS = {"selu": SELU, "relu": RELU, "softmax": SOFTMAX, "tanh": TANH}
_NAMES = {v: k for k, v in _ACTIVATIONS.items()}


def parse_model(document: dict) -> Tuple[Network, str, dict]:
    """(network, mesh model name, geometry dict) from a loaded YAML document."""
    if not isinstance(document, dict) or "network" not in document:
        raise ValueError("model file has no 'network' entry")
    network: Network = []
    width = 4
    for g, group in enumerate(document["network"]):
        layers = []
        for l, layer in enumerate(group):
            name = str(layer["activation"]).lower()
            if name not in _ACTIVATIONS:
                # example/load_model.hpp:33: "Unknown activation function"
                raise ValueError(f"Unknown activation function {layer['activation']}")
            w = np.asarray(layer["weights"], dtype=np.float32)
            b = np.asarray(layer["biases"], dtype=np.float32)
            if w.ndim != 2 or b.ndim != 1 or w.shape[1] != b.shape[0]:
                raise ValueError(f"group {g} layer {l}: weights must be [n_in][n_out] and biases [n_out]")
            if l == 0 and w.shape[0] % width != 0:
                raise ValueError(f"group {g}: {w.shape[0]} weight rows are not a multiple of the previous width {width}")
            if l > 0 and w.shape[0] != width:
                raise ValueError(f"group {g} layer {l}: {w.shape[0]} weight rows, previous width {width}")
            layers.append(Layer(np.ascontiguousarray(w), np.ascontiguousarray(b), _ACTIVATIONS[name]))
            width = b.shape[0]
        network.append(layers)
    return network, str(document.get("mesh", "")), dict(document.get("geometry", {}) or {})


def load_model(path: str) -> Tuple[Network, str, dict]:
    with open(path) as f:
        return parse_model(yaml.safe_load(f))


def n_neighbours_of(network: Network) -> int:
    """N from the first layer's row count: rows = (N + 1) * 4."""
    return network[0][0].weights.shape[0] // 4 - 1


def save_model(path: str, network: Network, mesh: str = "RING6", geometry: dict = None) -> None:
    doc = {
        "geometry": geometry or {},
        "mesh": mesh,
        "network": [[{"activation": _NAMES[int(layer.activation)],
                      "biases": [float(v) for v in layer.biases],
                      "weights": [[float(v) for v in row] for row in layer.weights]} for layer in group]
                    for group in network],
    }
    with open(path, "w") as f:
        yaml.safe_dump(doc, f, default_flow_style=None)
