"""Builder for pyc_ir_module values (the IR of PyC's include/pyc/ir.h).

Mirrors what PyC's C callers do by hand with pyc_ir_module_init /
pyc_ir_add_op (src/compiler/ir/ir.c:8-35): ops are appended in order, inputs
must reference earlier ops (ir.c:80-89).
"""
from . import abi


class ModuleBuilder:
    def __init__(self):
        self.module = abi.IrModule()
        self.module.op_count = 0

    def _add(self, kind, name, dtype, shape, inputs=()):
        m = self.module
        if m.op_count >= abi.PYC_IR_MAX_OPS:
            raise ValueError("module is full (PYC_IR_MAX_OPS)")
        idx = int(m.op_count)
        for i in inputs:
            if not (0 <= i < idx):
                raise ValueError(f"op {name}: input id {i} does not reference an earlier op")
        op = m.ops[idx]
        op.kind = kind
        op.name = name.encode()[: abi.PYC_IR_MAX_NAME - 1]
        op.dtype = dtype
        op.shape = abi.Shape.of(shape)
        for j, i in enumerate(inputs):
            op.input_ids[j] = i
        op.input_count = len(inputs)
        m.op_count = idx + 1
        return idx

    def _shape(self, i):
        return self.module.ops[i].shape.tolist()

    def _dtype(self, i):
        return int(self.module.ops[i].dtype)

    def input(self, name, dtype, shape):
        return self._add(abi.OP_INPUT, name, dtype, shape)

    def matmul(self, a, b, name=None):
        sa, sb = self._shape(a), self._shape(b)
        if len(sa) != 2 or len(sb) != 2 or sa[1] != sb[0]:
            raise ValueError(f"matmul shapes {sa} x {sb}")
        return self._add(abi.OP_MATMUL, name or f"matmul_{self.module.op_count}", self._dtype(a), [sa[0], sb[1]], (a, b))

    def add(self, a, b, name=None):
        return self._add(abi.OP_ADD, name or f"add_{self.module.op_count}", self._dtype(a), self._shape(a), (a, b))

    def relu(self, a, name=None):
        return self._add(abi.OP_RELU, name or f"relu_{self.module.op_count}", self._dtype(a), self._shape(a), (a,))

    def gelu(self, a, name=None):
        return self._add(abi.OP_GELU, name or f"gelu_{self.module.op_count}", self._dtype(a), self._shape(a), (a,))

    def layernorm(self, a, gamma=None, beta=None, name=None):
        ins = (a,) + ((gamma,) if gamma is not None else ()) + ((beta,) if beta is not None else ())
        return self._add(abi.OP_LAYERNORM, name or f"ln_{self.module.op_count}", self._dtype(a), self._shape(a), ins)

    def reduce_sum(self, a, name=None):
        s = self._shape(a)
        return self._add(abi.OP_REDUCE_SUM, name or f"rsum_{self.module.op_count}", self._dtype(a), s[:-1] or [1], (a,))

    def extended(self, name, dtype, shape, inputs):
        """An op PyC's IR has no kind for, carried by a REDUCE_SUM op whose name starts with "b200." and whose declared
        shape is its output shape (the backend's name-keyed side table): b200.softmax, b200.attention[.causal],
        b200.conv2d.p<ph>x<pw>.s<sh>x<sw>[.relu], b200.ffn_fp8."""
        if not name.startswith("b200."):
            raise ValueError("extended op names start with 'b200.'")
        return self._add(abi.OP_REDUCE_SUM, name, dtype, shape, tuple(inputs))

    def output(self, a, name=None):
        return self._add(abi.OP_OUTPUT, name or f"out_{self.module.op_count}", self._dtype(a), self._shape(a), (a,))


def matmul_bias_act(dtype, m, k, n, bias="row", act="relu"):
    """The chain PyC's GPU path accepts (cuda_backend.c:1232-1390) plus GELU:
    X[m,k] * W[k,n] (+ bias) (-> relu|gelu) -> output."""
    b = ModuleBuilder()
    x = b.input("x", dtype, [m, k])
    w = b.input("w", dtype, [k, n])
    cur = b.matmul(x, w)
    if bias == "row":
        cur = b.add(cur, b.input("b", dtype, [n]))
    elif bias == "matrix":
        cur = b.add(cur, b.input("b", dtype, [m, n]))
    elif bias == "scalar":
        cur = b.add(cur, b.input("b", dtype, [1]))
    if act == "relu":
        cur = b.relu(cur)
    elif act == "gelu":
        cur = b.gelu(cur)
    b.output(cur)
    return b.module
