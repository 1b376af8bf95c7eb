"""ONNX operators as objects.

Parity: crates/axonml-onnx/src/operators.rs (``OnnxOperator`` with ``execute(inputs) -> outputs``
and ``name``; one class per operator -- ``ReluOp``, ``GemmOp``, ``ConvOp``, ``ClipOp`` ... --, the
ones with attributes built by ``from_node``; ``create_operator(node)``, which fails with an
unsupported-operator error for anything else).  The arithmetic is the table ``model._OPS`` that
``OnnxModel.forward`` interprets graphs with, so an operator object and the interpreter cannot
disagree; inputs and outputs are torch tensors on whatever device the inputs live on."""
from __future__ import annotations

from .messages import NodeProto
from .model import _OPS, CompiledOp, OnnxError


class UnsupportedOperator(OnnxError, NotImplementedError):
    def __init__(self, op_type: str):
        super().__init__(f"Unsupported operator: {op_type}")
        self.op_type = op_type


class OnnxOperator:
    """One node's computation.  ``OP_TYPE`` names the ONNX operator, ``ARITY`` the (minimum,
    maximum) number of inputs it takes."""
    OP_TYPE = ""
    ARITY = (1, 1)

    def __init__(self, **attrs):
        self.attrs = {k: v for k, v in attrs.items() if v is not None}

    @classmethod
    def from_node(cls, node):
        """Operator with the attributes of a ``NodeProto`` (or of an interpreter ``CompiledOp``)."""
        return cls(**(node.attrs() if isinstance(node, NodeProto) else dict(node.attrs)))

    def name(self) -> str:
        return self.OP_TYPE

    def execute(self, inputs) -> list:
        """``inputs``: tensors, ``None`` for an omitted optional input.  Returns the list of outputs."""
        inputs = list(inputs)
        lo, hi = self.ARITY
        given = len(inputs)
        if given < lo or (hi is not None and given > hi):
            want = f"{lo}" if hi == lo else f"{lo} to {hi}" if hi is not None else f"at least {lo}"
            raise OnnxError(f"{self.OP_TYPE} takes {want} inputs, got {given}")
        if any(t is None for t in inputs[:lo]):
            raise OnnxError(f"{self.OP_TYPE}: a required input is missing")
        out = _OPS[self.OP_TYPE](inputs, self.attrs)
        return list(out) if isinstance(out, (tuple, list)) else [out]

    __call__ = execute

    def __repr__(self) -> str:
        return f"{type(self).__name__}({', '.join(f'{k}={v!r}' for k, v in self.attrs.items())})"


def _op(class_name: str, op_type: str, arity, doc: str):
    return type(class_name, (OnnxOperator,), {"OP_TYPE": op_type, "ARITY": arity, "__doc__": doc})


ReluOp = _op("ReluOp", "Relu", (1, 1), "max(x, 0)")
SigmoidOp = _op("SigmoidOp", "Sigmoid", (1, 1), "1 / (1 + exp(-x))")
TanhOp = _op("TanhOp", "Tanh", (1, 1), "tanh(x)")
SoftmaxOp = _op("SoftmaxOp", "Softmax", (1, 1), "softmax over ``axis`` (default -1)")
LeakyReluOp = _op("LeakyReluOp", "LeakyRelu", (1, 1), "x for x > 0, ``alpha`` * x otherwise (alpha 0.01)")
GeluOp = _op("GeluOp", "Gelu", (1, 1), "GELU; ``approximate='tanh'`` selects the tanh form")
AddOp = _op("AddOp", "Add", (2, 2), "a + b with broadcasting")
SubOp = _op("SubOp", "Sub", (2, 2), "a - b with broadcasting")
MulOp = _op("MulOp", "Mul", (2, 2), "a * b with broadcasting")
DivOp = _op("DivOp", "Div", (2, 2), "a / b with broadcasting")
MatMulOp = _op("MatMulOp", "MatMul", (2, 2), "matrix product with batch broadcasting")
GemmOp = _op("GemmOp", "Gemm", (2, 3), "alpha * op(A) op(B) + beta * C with ``transA`` / ``transB``")
SqrtOp = _op("SqrtOp", "Sqrt", (1, 1), "square root")
PowOp = _op("PowOp", "Pow", (2, 2), "base ** exponent")
ExpOp = _op("ExpOp", "Exp", (1, 1), "e ** x")
LogOp = _op("LogOp", "Log", (1, 1), "natural logarithm")
ReshapeOp = _op("ReshapeOp", "Reshape", (2, 2), "reshape to the int64 shape input; 0 copies the extent, -1 is inferred")
TransposeOp = _op("TransposeOp", "Transpose", (1, 1), "permute by ``perm`` (reversed dimensions without it)")
FlattenOp = _op("FlattenOp", "Flatten", (1, 1), "2-D view split at ``axis`` (default 1)")
SqueezeOp = _op("SqueezeOp", "Squeeze", (1, 2), "drop dimensions of extent 1 (``axes`` attribute or input)")
UnsqueezeOp = _op("UnsqueezeOp", "Unsqueeze", (1, 2), "insert dimensions of extent 1 at ``axes``")
ConcatOp = _op("ConcatOp", "Concat", (1, None), "concatenate along ``axis``")
GatherOp = _op("GatherOp", "Gather", (2, 2), "index along ``axis``")
ReduceSumOp = _op("ReduceSumOp", "ReduceSum", (1, 2), "sum over ``axes`` with ``keepdims`` (default 1)")
ReduceMeanOp = _op("ReduceMeanOp", "ReduceMean", (1, 2), "mean over ``axes`` with ``keepdims``")
ReduceMaxOp = _op("ReduceMaxOp", "ReduceMax", (1, 2), "maximum over ``axes`` with ``keepdims``")
ConvOp = _op("ConvOp", "Conv", (2, 3), "2-D convolution with ``strides``, ``pads``, ``dilations``, ``group``")
MaxPoolOp = _op("MaxPoolOp", "MaxPool", (1, 1), "2-D max pooling with ``kernel_shape``, ``strides``, ``pads``")
AvgPoolOp = _op("AvgPoolOp", "AveragePool", (1, 1), "2-D average pooling with ``kernel_shape``, ``strides``, ``pads``")
BatchNormOp = _op("BatchNormOp", "BatchNormalization", (5, 5), "inference batch norm: x, scale, bias, mean, var; ``epsilon``")
DropoutOp = _op("DropoutOp", "Dropout", (1, 3), "identity (inference)")
ConstantOp = _op("ConstantOp", "Constant", (0, 0), "the ``value`` tensor (or ``value_float`` / ``value_int``)")
IdentityOp = _op("IdentityOp", "Identity", (1, 1), "x")
CastOp = _op("CastOp", "Cast", (1, 1), "convert to the element type ``to``")
ShapeOp = _op("ShapeOp", "Shape", (1, 1), "the shape as an int64 vector")
EqualOp = _op("EqualOp", "Equal", (2, 2), "a == b")
GreaterOp = _op("GreaterOp", "Greater", (2, 2), "a > b")
LessOp = _op("LessOp", "Less", (2, 2), "a < b")
ClipOp = _op("ClipOp", "Clip", (1, 3), "clamp to [min, max] from attributes or inputs")
# beyond the reference's set
GlobalAveragePoolOp = _op("GlobalAveragePoolOp", "GlobalAveragePool", (1, 1), "mean over the spatial dimensions")
NegOp = _op("NegOp", "Neg", (1, 1), "-x")
AbsOp = _op("AbsOp", "Abs", (1, 1), "|x|")
ErfOp = _op("ErfOp", "Erf", (1, 1), "error function")
WhereOp = _op("WhereOp", "Where", (3, 3), "condition ? a : b")
LayerNormOp = _op("LayerNormOp", "LayerNormalization", (2, 3), "layer norm from ``axis`` on; ``epsilon``")

OPERATOR_CLASSES = {c.OP_TYPE: c for c in list(globals().values()) if isinstance(c, type) and issubclass(c, OnnxOperator) and c.OP_TYPE}
assert set(OPERATOR_CLASSES) == set(_OPS), sorted(set(_OPS) ^ set(OPERATOR_CLASSES))


def create_operator(node) -> OnnxOperator:
    """Operator object for a ``NodeProto`` or ``CompiledOp``; raises ``UnsupportedOperator`` otherwise."""
    op_type = node.op_type
    cls = OPERATOR_CLASSES.get(op_type)
    if cls is None:
        raise UnsupportedOperator(op_type)
    return cls.from_node(node)


__all__ = ["OnnxOperator", "UnsupportedOperator", "create_operator", "OPERATOR_CLASSES", "CompiledOp"] + [c.__name__ for c in OPERATOR_CLASSES.values()]
