"""The seven MatMulNBits nodes of a Llama-3-8B-shaped decoder layer as one driver.

A decoder layer multiplies four different activations by seven weight matrices: the attention
input by q, k and v, the attention output by o, the MLP input by gate and up, the gated
intermediate by down. Nodes that take the same activations go through
``matmul_device_group`` (one call: whatever the nodes share - the staged or quantized
activations, at one token the kernel launch itself - is done once); o and down are single
calls. The driver owns the weights and the output buffers; what happens between the
projections (attention, the gate's activation function) is the caller's.

Shapes follow onnx-light's Qwen3 / Llama inference notes
(docs/next_steps/2026/2026_08_qwen3_inference.rst:374-380): q 4096->4096, k and v 4096->1024,
o 4096->4096, gate and up 4096->14336, down 14336->4096.
"""

from __future__ import annotations

from . import synthetic as syn

#: stage name -> (name of the activations it takes, nodes that take them)
STAGES = (
    ("attn_in", ("q", "k", "v")),
    ("attn_out", ("o",)),
    ("mlp_in", ("gate", "up")),
    ("mlp_mid", ("down",)),
)


class DecoderLayerProjections:
    """Weights of the seven nodes on one GPU and the four calls that run them.

    ``cases`` maps node name to a :class:`synthetic.Case` (or anything with ``b``, ``scales``,
    ``zero_points``, ``bias``, ``k``, ``n``, ``bits``, ``block_size``)."""

    def __init__(self, cases: dict, device: int = 0):
        import torch

        from .. import MatMulNBitsWeights

        self.device = device
        self.cases = dict(cases)
        self.nodes = {}
        for _, names in STAGES:
            for name in names:
                case = self.cases[name]
                self.nodes[name] = MatMulNBitsWeights(
                    case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n, bits=case.bits,
                    block_size=case.block_size, device=device)
        self._torch = torch
        self._outputs = {}

    @classmethod
    def synthetic(cls, m: int = 16, accuracy_level: int = 0, device: int = 0):
        """The layer of benchmark configuration 4 (4-bit, block_size 32, no zero points)."""
        cases = {case.name.removeprefix("cfg4_"): case for case in syn.config4(accuracy_level, m)}
        return cls(cases, device)

    def inputs_from_cases(self) -> dict:
        """Device activations for the four stages, taken from the first node of each stage."""
        torch = self._torch
        return {key: torch.from_numpy(self.cases[names[0]].a).to(f"cuda:{self.device}")
                for key, names in STAGES}

    def outputs(self, m: int) -> dict:
        """Output buffers [m, N] per node, allocated once per M."""
        torch = self._torch
        if m not in self._outputs:
            self._outputs[m] = {name: torch.empty((m, node.n), dtype=torch.float32, device=f"cuda:{self.device}")
                                for name, node in self.nodes.items()}
        return self._outputs[m]

    def algorithmic_bytes(self, m: int) -> int:
        """Bytes the seven nodes must move once: every node's operands, A and Y counted per node."""
        return sum(node.algorithmic_bytes(m) for node in self.nodes.values())

    def run(self, inputs: dict, accuracy_level: int = 0, stream=None, grouped: bool = True) -> dict:
        """Launches the seven projections (asynchronously) and returns their output tensors.
        ``inputs``: the four activation tensors by stage key. ``grouped=False`` runs node by node."""
        from ..matmul_nbits import matmul_device_group

        m = int(inputs[STAGES[0][0]].shape[0])
        outs = self.outputs(m)
        for key, names in STAGES:
            a = inputs[key]
            if grouped:
                matmul_device_group([self.nodes[n] for n in names], a, [outs[n] for n in names],
                                    accuracy_level=accuracy_level, stream=stream)
            else:
                for n in names:
                    self.nodes[n].matmul_device(a, outs[n], accuracy_level=accuracy_level, stream=stream)
        return outs

    def poll_status(self) -> int:
        """First non-zero device status word of any node (0 = fine)."""
        for node in self.nodes.values():
            status = node.poll_status()
            if status != 0:
                return status
        return 0

    def close(self) -> None:
        for node in self.nodes.values():
            node.close()
        self.nodes = {}
        self._outputs = {}
