"""Model and property ingestion for the bound-propagation path: the NNet text format and a VNN-LIB 1.0 subset.

NNet (crates/ny-onnx/src/nnet/parser.rs): comment lines start with `//`; a header line
`numLayers, inputSize, outputSize, maxLayerSize`, the layer sizes, one unused line, input minimums, input
maximums, means (inputs, optionally one more for the output), ranges (same), then per layer its weight rows
(`out` lines of `in` values) followed by its biases (one per line).  Every hidden layer is followed by a ReLU.
Properties are stated in the network's own input space, so the weights are used as they are.

VNN-LIB subset (crates/ny-onnx/src/vnnlib): `(declare-const X_i Real)`, `(declare-const Y_j Real)`, and `assert`s
built from `<=`, `>=`, `and`, `or` over `X_i`, `Y_j` and numeric constants.  Input asserts give the box; the output
asserts describe the VIOLATION (the standard convention: the verifier must show it cannot be reached).  The output
side is returned in disjunctive normal form: a list of conjunctions of atoms `c . y + d >= 0`.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field

import numpy as np

from .engine import EngineError, Network

_INVALID = 3  # NYB200_ERR_INVALID_SPEC


@dataclass
class NNet:
    layer_sizes: list
    weights: list
    biases: list
    input_minimums: np.ndarray
    input_maximums: np.ndarray
    input_means: np.ndarray
    input_ranges: np.ndarray
    output_mean: float = 0.0
    output_range: float = 1.0

    def to_network(self) -> Network:
        return Network(self.weights, self.biases)


def _csv(line: str, conv):
    return [conv(t.strip()) for t in line.split(",") if t.strip()]


def parse_nnet(text: str) -> NNet:
    lines = [ln for ln in text.splitlines() if ln.strip() and not ln.startswith("//")]
    it = iter(lines)

    def need(what):
        try:
            return next(it)
        except StopIteration:
            raise EngineError(_INVALID, f"nnet: missing {what}") from None

    header = _csv(need("header line"), int)
    if len(header) < 4:
        raise EngineError(_INVALID, f"nnet: header has {len(header)} values, expected 4")
    num_layers, input_size, output_size = header[0], header[1], header[2]
    sizes = _csv(need("layer sizes"), int)
    if len(sizes) != num_layers + 1:
        raise EngineError(_INVALID, f"nnet: expected {num_layers + 1} layer sizes, got {len(sizes)}")
    if sizes[0] != input_size or sizes[-1] != output_size:
        raise EngineError(_INVALID, "nnet: layer sizes disagree with the header")
    need("symmetric flag")
    mins = np.array(_csv(need("input minimums"), float), np.float32)
    maxs = np.array(_csv(need("input maximums"), float), np.float32)
    means = _csv(need("means"), float)
    ranges = _csv(need("ranges"), float)
    out_mean = means[input_size] if len(means) > input_size else 0.0
    out_range = ranges[input_size] if len(ranges) > input_size else 1.0
    weights, biases = [], []
    for k in range(num_layers):
        n_in, n_out = sizes[k], sizes[k + 1]
        rows = []
        for _ in range(n_out):
            vals = _csv(need("weight row"), float)
            if len(vals) < n_in:
                raise EngineError(_INVALID, f"nnet: weight row has {len(vals)} values, expected {n_in}")
            rows.append(vals[:n_in])
        weights.append(np.array(rows, np.float32).reshape(n_out, n_in))
        b = []
        for _ in range(n_out):
            try:
                b.append(float(need("bias value").strip().rstrip(",")))
            except ValueError as e:
                raise EngineError(_INVALID, f"nnet: invalid bias value: {e}") from None
        biases.append(np.array(b, np.float32))
    return NNet(sizes, weights, biases, mins, maxs, np.array(means[:input_size], np.float32),
                np.array(ranges[:input_size], np.float32), float(out_mean), float(out_range))


def write_nnet(weights, biases) -> str:
    """The inverse of parse_nnet for a plain ReLU MLP (unit input range, no normalisation)."""
    sizes = [int(weights[0].shape[1])] + [int(w.shape[0]) for w in weights]
    out = ["// NNet written by ny_b200.formats.write_nnet",
           ",".join(str(v) for v in (len(weights), sizes[0], sizes[-1], max(sizes))) + ",",
           ",".join(str(v) for v in sizes) + ",", "0,",
           ",".join("0.0" for _ in range(sizes[0])) + ",", ",".join("1.0" for _ in range(sizes[0])) + ",",
           ",".join("0.0" for _ in range(sizes[0] + 1)) + ",", ",".join("1.0" for _ in range(sizes[0] + 1)) + ","]
    for w, b in zip(weights, biases):
        for row in np.asarray(w, np.float32):
            out.append(",".join(repr(float(v)) for v in row) + ",")
        for v in np.asarray(b, np.float32):
            out.append(repr(float(v)) + ",")
    return "\n".join(out) + "\n"


# ------------------------------------------------------------------------------------------- VNN-LIB
@dataclass
class Atom:
    """c . y + d >= 0 over the network outputs."""
    c: np.ndarray
    d: float


@dataclass
class Property:
    in_lo: np.ndarray
    in_hi: np.ndarray
    violation: list = field(default_factory=list)  # disjunction (list) of conjunctions (lists) of Atoms


def _tokens(text: str):
    text = re.sub(r";[^\n]*", "", text)
    return re.findall(r"\(|\)|[^\s()]+", text)


def _sexprs(tokens):
    stack, out = [], []
    for t in tokens:
        if t == "(":
            stack.append([])
        elif t == ")":
            if not stack:
                raise EngineError(_INVALID, "vnnlib: unbalanced parenthesis")
            done = stack.pop()
            (stack[-1] if stack else out).append(done)
        else:
            if not stack:
                raise EngineError(_INVALID, f"vnnlib: token outside an expression: {t}")
            stack[-1].append(t)
    if stack:
        raise EngineError(_INVALID, "vnnlib: unbalanced parenthesis")
    return out


def _term(t, n_in, n_out):
    """('x', i, None) / ('y', j, None) / ('const', None, value)"""
    if isinstance(t, list):
        raise EngineError(1, "vnnlib: arithmetic terms are outside the supported subset")
    m = re.fullmatch(r"([XY])_(\d+)", t)
    if m:
        idx = int(m.group(2))
        if idx >= (n_in if m.group(1) == "X" else n_out):
            raise EngineError(_INVALID, f"vnnlib: {t} out of range")
        return ("x" if m.group(1) == "X" else "y", idx, None)
    try:
        return ("const", None, float(t))
    except ValueError:
        raise EngineError(_INVALID, f"vnnlib: unknown term {t}") from None


def _dnf(expr, n_in, n_out, box, under_or=False):
    """Disjunctive normal form of an output expression; input atoms tighten `box` in place and drop out.
    An input atom anywhere below an `or` would make the input set a union of boxes (the reference keeps one box
    per disjunct, crates/ny-onnx/src/vnnlib/parser.rs:384,438); tightening the one shared box with it would
    intersect the disjuncts' boxes and could certify a property that fails elsewhere in the union, so it is
    declined."""
    op = expr[0]
    if op == "and":
        parts = [_dnf(e, n_in, n_out, box, under_or) for e in expr[1:]]
        acc = [[]]
        for part in parts:
            if part is None:
                continue
            acc = [a + b for a in acc for b in part]
        return acc
    if op == "or":
        out = []
        for e in expr[1:]:
            part = _dnf(e, n_in, n_out, box, True)
            if part is None:
                raise EngineError(1, "vnnlib: input constraints inside a disjunction are outside the supported subset")
            if any(len(c) == 0 for c in part):
                raise EngineError(1, "vnnlib: a disjunct without output constraints is outside the supported subset")
            out.extend(part)
        return out
    if op in ("<=", ">="):
        if len(expr) != 3:
            raise EngineError(_INVALID, "vnnlib: comparison needs two operands")
        a, b = _term(expr[1], n_in, n_out), _term(expr[2], n_in, n_out)
        if op == "<=":  # a <= b  <=>  b >= a
            a, b = b, a
        # now: a >= b
        kinds = (a[0], b[0])
        if "x" in kinds:
            if under_or:
                raise EngineError(1, "vnnlib: input constraints inside a disjunction are outside the supported subset")
            if kinds == ("x", "const"):
                box[0][a[1]] = max(box[0][a[1]], b[2])
            elif kinds == ("const", "x"):
                box[1][b[1]] = min(box[1][b[1]], a[2])
            else:
                raise EngineError(1, "vnnlib: relations between inputs are outside the supported subset")
            return None
        c = np.zeros(n_out, np.float32)
        d = 0.0
        for sign, t in ((1.0, a), (-1.0, b)):
            if t[0] == "y":
                c[t[1]] += sign
            else:
                d += sign * t[2]
        return [[Atom(c, float(d))]]
    raise EngineError(1, f"vnnlib: operator {op} is outside the supported subset")


def parse_vnnlib(text: str, n_in: int, n_out: int) -> Property:
    box = [np.full(n_in, -np.inf, np.float64), np.full(n_in, np.inf, np.float64)]
    clauses = [[]]
    for e in _sexprs(_tokens(text)):
        if not e:
            continue
        if e[0] == "declare-const":
            continue
        if e[0] != "assert" or len(e) != 2:
            raise EngineError(1, f"vnnlib: statement {e[0]} is outside the supported subset")
        part = _dnf(e[1], n_in, n_out, box)
        if part is None:
            continue
        clauses = [a + b for a in clauses for b in part]   # top-level asserts are a conjunction
    if not np.all(np.isfinite(box[0])) or not np.all(np.isfinite(box[1])):
        raise EngineError(_INVALID, "vnnlib: every input needs a lower and an upper bound")
    if np.any(box[0] > box[1]):
        raise EngineError(_INVALID, "vnnlib: empty input box")
    clauses = [c for c in clauses if c]
    if not clauses:
        # no output atom at all: the violation set would be the whole box, not the empty set
        raise EngineError(1, "vnnlib: a property without output constraints is outside the supported subset")
    # the fp32 box must contain the stated one: round the ends outward
    lo32, hi32 = box[0].astype(np.float32), box[1].astype(np.float32)
    lo32 = np.where(lo32.astype(np.float64) > box[0], np.nextafter(lo32, np.float32(-np.inf)), lo32).astype(np.float32)
    hi32 = np.where(hi32.astype(np.float64) < box[1], np.nextafter(hi32, np.float32(np.inf)), hi32).astype(np.float32)
    return Property(lo32, hi32, clauses)
