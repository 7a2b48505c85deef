"""Generates tests/golden/ls_kat.npz: answers computed FROM THE REFERENCE'S OWN KERNEL TEXT.

The reference's kernels for the DeltaNet recurrence, decay gate, convolution, sigmoid / SiLU and RoPE
exist only as `.ls` sources (inference/*.ls); its interpreters cannot evaluate them and its compiler
emits sm_90 opcodes.  Its Python front end (bootstrap-py/lexer.py, parser.py) does parse them.  This
script imports that parser from the reference tree, and evaluates the resulting syntax trees with a
small lock-step SIMT interpreter (one numpy lane per GPU thread, float32 arithmetic), so the fixture pins
the C oracle (oracle/oracle.c) to what the reference text says, statement by statement.

    LITHOS_REF=<reference checkout> python tests/golden/make_ls_golden.py

Intrinsic meanings follow the reference's code generator (bootstrap-py/codegen.py:431-475):
`exp d s` = 2^s (MUFU.EX2), `lg d s` = log2 s (MUFU.LG2), `rcp`, `rsqrt`, `sqrt`, `sin`, `cos`, `neg d s` = 0 - s;
`fma d a b c` = a*b+c with one rounding; `mad d a b c` = a*b+c on integers; `shl/shr/and/add/mul d a b`.
The special-function units' approximation error is not modelled (exact float32 results are stored; the
tolerance in the test absorbs it).

Kernels evaluated (file:lines in the reference):
  inference/decay_gate.ls:28-57 decay_gate        inference/deltanet_fused.ls:37-151 deltanet_fused
  inference/delta_update.ls:24-54 delta_update    inference/recur.ls:12-40 conv1d_infer, :45-55 gate_sigmoid
  inference/elementwise.ls:7-34 residual_add, elemwise_mul, activate_silu, scale
  inference/attend.ls:21-71 rope
Not evaluated: attention_score (attend.ls:85-191; this build's primary attention contract differs from that
text on purpose: natural exp and a true -inf start) and the shuffle-based reductions of reduce.ls.
"""
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import ls_inputs as I  # noqa: E402

REF = os.environ.get("LITHOS_REF")
if not REF or not (Path(REF) / "bootstrap-py" / "parser.py").exists():
    sys.exit("set LITHOS_REF to a checkout of the reference (its bootstrap-py parser is imported from there)")
sys.path.insert(0, str(Path(REF) / "bootstrap-py"))
from bridge import lex_and_convert  # noqa: E402  (reference module)
import parser as P  # noqa: E402  (reference module)

F32 = np.float32


def parse_kernel(ls_file: str, name: str):
    src = (Path(REF) / "inference" / ls_file).read_text(encoding="utf-8")
    for fn in P.Parser(lex_and_convert(src)).parse():
        if isinstance(fn, P.FuncDef) and fn.name == name:
            return fn
    raise KeyError(f"{name} not found in {ls_file}")


def is_int(a) -> bool:
    return np.issubdtype(np.asarray(a).dtype, np.integer)


class LoopStart:
    def __init__(self, node):
        self.node = node


class LoopEnd:
    pass


def linearize(body):
    """The statements in source order with explicit loop brackets.  The kernel sources close every `for` with an
    `endfor`.  The reference's Python parser nests a loop's indented lines under the For node and keeps `endfor` as a
    statement of its own, but where a loop is the last statement of an enclosing loop's block it swallows that
    `endfor` and ends the enclosing block early (deltanet_fused.ls:97-109: the dumped tree puts everything after the
    first inner loop at function level).  Source order survives, so the structure the text states is recovered by
    bracket matching: a For whose next sibling is not an EndFor lost its `endfor` right after its parsed lines."""
    out = []
    for n, s in enumerate(body):
        if isinstance(s, P.For):
            out.append(LoopStart(s))
            out.extend(linearize(s.body))
            nxt = body[n + 1] if n + 1 < len(body) else None
            if nxt is not None and not isinstance(nxt, P.EndFor):
                out.append(LoopEnd())
        elif isinstance(s, P.EndFor):
            out.append(LoopEnd())
        else:
            out.append(s)
    return out


def check_balanced(items, name):
    depth = 0
    for s in items:
        depth += isinstance(s, LoopStart) - isinstance(s, LoopEnd)
        assert depth >= 0, f"{name}: endfor without for"
    assert depth == 0, f"{name}: {depth} loop(s) left open"


class Simt:
    """All threads of a launch advance one statement at a time (numpy arrays of length n_threads)."""

    def __init__(self, fn, buffers: dict, params: dict, n_threads: int, block: int):
        self.fn, self.buf, self.T, self.block = fn, buffers, n_threads, block
        self.env = {k: np.full(n_threads, v, dtype=np.int64 if isinstance(v, (int, np.integer)) else F32)
                    for k, v in params.items()}
        self.shared = {}
        self.tid = np.arange(n_threads, dtype=np.int64)
        self.alive = np.ones(n_threads, dtype=bool)
        check_balanced(linearize(fn.body), fn.name)
        missing = [p for p in fn.params if p not in buffers]
        assert not missing, f"{fn.name}: no buffer for {missing}"

    # ---- expressions ----
    def ev(self, e, mask):
        if isinstance(e, P.IntLit):
            return np.full(self.T, e.value, dtype=np.int64)
        if isinstance(e, P.FloatLit):
            return np.full(self.T, e.value, dtype=F32)
        if isinstance(e, P.Ident):
            return self.env[e.name]
        if isinstance(e, P.BinOp):
            return self.binop(e.op, self.ev(e.left, mask), self.ev(e.right, mask))
        if isinstance(e, P.ArrayIndex):
            return self.load(e.base.name, self.ev(e.index, mask), mask)
        if isinstance(e, P.FuncCall) and len(e.args) == 1:
            return self.unary(e.name, self.ev(e.args[0], mask))
        if isinstance(e, P.UnaryOp):
            return self.unary(e.op, self.ev(e.operand, mask))
        raise NotImplementedError(f"expression {e!r}")

    @staticmethod
    def binop(op, a, b):
        if is_int(a) and is_int(b):
            return {"+": a + b, "-": a - b, "*": a * b, "&": a & b, "|": a | b, "^": a ^ b,
                    "<<": a << b, ">>": a >> b}[op] if op != "/" else a // b
        a, b = a.astype(F32), b.astype(F32)
        if op == "+":
            return a + b
        if op == "-":
            return a - b
        if op == "*":
            return a * b
        if op == "/":
            return a / b
        raise NotImplementedError(op)

    @staticmethod
    def unary(name, s):
        s = s.astype(F32)
        with np.errstate(all="ignore"):
            if name in ("exp", "exp2"):
                return np.exp2(s).astype(F32)
            if name in ("lg", "lg2"):
                return np.log2(s).astype(F32)
            if name == "rcp":
                return (F32(1.0) / s).astype(F32)
            if name == "rsqrt":
                return (F32(1.0) / np.sqrt(s)).astype(F32)
            if name == "sqrt":
                return np.sqrt(s).astype(F32)
            if name == "sin":
                return np.sin(s).astype(F32)
            if name == "cos":
                return np.cos(s).astype(F32)
            if name == "neg":
                return (F32(0.0) - s).astype(F32)
        raise NotImplementedError(name)

    def load(self, name, idx, mask):
        idx = np.where(mask, idx, 0).astype(np.int64)
        if name in self.shared:
            return self.shared[name][self.tid // self.block, idx]
        flat = self.buf[name].reshape(-1)
        assert idx.max(initial=0) < flat.size, f"load {name}[{idx.max()}] out of range"
        return flat[idx]

    def store(self, name, idx, val, mask):
        if not mask.any():
            return
        idx = idx.astype(np.int64)
        if name in self.shared:
            self.shared[name][(self.tid // self.block)[mask], idx[mask]] = val[mask]
            return
        flat = self.buf[name].reshape(-1)
        assert idx[mask].max() < flat.size, f"store {name}[{idx[mask].max()}] out of range"
        flat[idx[mask]] = val[mask].astype(flat.dtype)

    def assign(self, name, val, mask):
        old = self.env.get(name)
        if old is None or old.dtype != val.dtype:
            old = np.zeros(self.T, dtype=val.dtype) if old is None else old.astype(val.dtype)
        self.env[name] = np.where(mask, val, old)

    @staticmethod
    def fma(a, b, c):
        # a*b is exact in float64 (24+24 significant bits), so the sum rounded once to float32 is the fused result
        # except in double-rounding corner cases far below the test tolerance
        return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(F32)

    # ---- statements ----
    def run(self):
        self.block_exec(linearize(self.fn.body), self.alive.copy())

    def uniform_int(self, e, mask):
        v = self.ev(e, mask)
        assert is_int(v) and (v[mask] == v[mask][0]).all(), "loop bounds must be uniform integers"
        return int(v[mask][0])

    def block_exec(self, body, mask):
        i = 0
        while i < len(body):
            s = body[i]
            mask = mask & self.alive
            if isinstance(s, (P.Param, P.Comment, P.Barrier)):
                pass        # parameters are preset; lock-step execution makes every barrier trivially satisfied
            elif isinstance(s, P.Each):
                self.env[s.var] = self.tid.copy()
            elif isinstance(s, P.Shared):
                n = s.count.value if isinstance(s.count, P.IntLit) else int(s.count)
                self.shared[s.name] = np.zeros(((self.T + self.block - 1) // self.block, n), dtype=F32)
            elif isinstance(s, P.Assignment):
                self.assign(s.target, self.ev(s.value, mask), mask)
            elif isinstance(s, P.ArrayStore):
                self.store(s.target, self.ev(s.index, mask), self.ev(s.value, mask), mask)
            elif isinstance(s, P.Fma):
                self.assign(s.dest, self.fma(self.ev(s.a, mask), self.ev(s.b, mask), self.ev(s.c, mask)), mask)
            elif isinstance(s, P.TypeCast):
                v = self.ev(s.src, mask)
                self.assign(s.dest, v.astype(F32) if s.to_type == "f32" else v.astype(np.int64), mask)
            elif isinstance(s, P.PrefixOp):
                op = {"shl": "<<", "shr": ">>", "and": "&", "or": "|", "xor": "^", "add": "+", "sub": "-", "mul": "*"}[s.op]
                self.assign(s.dest, self.binop(op, self.ev(s.a, mask), self.ev(s.b, mask)), mask)
            elif isinstance(s, P.FuncCall):
                if s.name == "mad" and len(s.args) == 4:
                    a, b, c = (self.ev(x, mask) for x in s.args[1:])
                    self.assign(s.args[0].name, a * b + c, mask)
                elif len(s.args) == 2:
                    self.assign(s.args[0].name, self.unary(s.name, self.ev(s.args[1], mask)), mask)
                else:
                    raise NotImplementedError(f"call {s!r}")
            elif isinstance(s, P.If):
                a, b = self.ev(s.left, mask), self.ev(s.right, mask)
                cond = {"==": a == b, "!=": a != b, ">=": a >= b, "<": a < b, ">": a > b, "<=": a <= b}[s.op]
                if s.label == "exit" and not s.body:
                    self.alive &= ~(mask & cond)
                else:
                    self.block_exec(linearize(s.body), mask & cond)
                    if s.else_body:
                        self.block_exec(linearize(s.else_body), mask & ~cond)
            elif isinstance(s, LoopStart):
                depth, j = 1, i + 1            # the matching end of this loop
                while depth:
                    depth += isinstance(body[j], LoopStart) - isinstance(body[j], LoopEnd)
                    j += 1
                f = s.node
                lo, hi, st = (self.uniform_int(x, mask) for x in (f.start, f.end, f.step))
                for it in range(lo, hi, st):
                    self.env[f.var] = np.full(self.T, it, dtype=np.int64)
                    self.block_exec(body[i + 1:j - 1], mask)
                i = j - 1
            else:
                raise NotImplementedError(f"statement {s!r}")
            i += 1


def launch(ls_file, name, buffers, params, n_threads, block):
    sim = Simt(parse_kernel(ls_file, name), buffers, params, n_threads, block)
    sim.run()
    return sim


def main():
    out = {}
    # ---- decay_gate (text as written: softplus through lg = log2) ----
    c = I.decay_gate_case()
    dec = np.zeros(48, F32)
    launch("decay_gate.ls", "decay_gate", dict(a_proj=c["a_proj"], a_log=c["a_log"], dt_bias=c["dt_bias"], decay=dec),
           dict(N=48), 64, 64)
    out["decay_gate_text"] = dec
    beta = np.zeros(48, F32)
    launch("recur.ls", "gate_sigmoid", dict(logit=c["b"], beta=beta), dict(N=48), 64, 64)
    out["gate_sigmoid"] = beta

    # ---- deltanet_fused: two tokens, state carried ----
    c = I.deltanet_fused_case()
    state = c["state"].copy()
    outs = np.zeros((c["T"], c["HV"], c["d"]), F32)
    for t in range(c["T"]):
        launch("deltanet_fused.ls", "deltanet_fused",
               dict(q=c["q"][t].copy(), k=c["k"][t].copy(), v=c["v"][t].copy(), z=c["z"][t].copy(), decay=c["decay"][t].copy(),
                    beta=c["beta"][t].copy(), state=state, output=outs[t]), dict(d=c["d"], gqa=3), c["HK"] * 128, 128)
    out["dnf_out"] = outs
    out["dnf_state_rows"] = state[:, [0, 5, 77, 127], :].copy()
    out["dnf_state_sum"] = state.astype(np.float64).sum(axis=(1, 2))

    # ---- delta_update: one head, no read-out ----
    c = I.delta_update_case()
    s_out = np.zeros_like(c["state"])
    launch("delta_update.ls", "delta_update", dict(state=c["state"].copy(), k=c["k"], v=c["v"], state_out=s_out),
           dict(d=c["d"], beta=float(c["beta"]), decay=float(c["decay"])), 32, 32)
    out["du_state"] = s_out

    # ---- conv1d_infer: five tokens through the 3-deep history ----
    c = I.conv1d_case()
    hist = c["hist"].copy()
    ys = np.zeros((c["T"], c["C"]), F32)
    for t in range(c["T"]):
        launch("recur.ls", "conv1d_infer", dict(x=c["x"][t].copy(), weights=c["w"].copy(), state=hist, output=ys[t]),
               dict(N=c["C"]), 128, 128)
    out["conv_y"] = ys
    out["conv_hist"] = hist

    # ---- elementwise ----
    c = I.elementwise_case()
    n = c["a"].size
    for name, bufs in (("residual_add", dict(a=c["a"], b=c["b"])), ("elemwise_mul", dict(a=c["a"], b=c["b"])),
                       ("scale", dict(x=c["a"], factor=c["b"])), ("activate_silu", dict(x=c["a"]))):
        o = np.zeros(n, F32)
        launch("elementwise.ls", name, dict(output=o, **{k: v.copy() for k, v in bufs.items()}), {}, n, 256)
        out["ew_" + name] = o

    # ---- rope: one head of 256 (128 pair lanes), q and k together ----
    c = I.rope_case()
    qo, ko = np.zeros(256, F32), np.zeros(256, F32)
    launch("attend.ls", "rope", dict(q=c["q"].copy(), k=c["k"].copy(), q_out=qo, k_out=ko),
           dict(d_head=c["d_head"], pos=c["pos"]), 128, 128)
    out["rope_q"], out["rope_k"] = qo, ko

    path = HERE / "ls_kat.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes):", ", ".join(f"{k}{list(v.shape)}" for k, v in out.items()))


if __name__ == "__main__":
    main()
