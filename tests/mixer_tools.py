"""Helpers of the device tests that run one mixer with a cache manager of its own: sequences fed in
portions, several a step, slots and pages given back and used again."""
import pytest
import torch


def close(got, want, dtype, f32=2e-5, bf16=2.5e-2):
    want = torch.as_tensor(want).double()
    err = float((got.double().cpu() - want).abs().max() / want.abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16), f"relative error {err:.2e}"
    return err


def bf(t):
    """Values that are exact in bfloat16, as float64."""
    return t.to(torch.bfloat16).double()


def make_kit():
    from gollmgo_b200 import parts
    from gollmgo_b200.cache import CacheManager
    from gollmgo_b200.csrc import ops
    from gollmgo_b200.engine.batch import BatchBuilder, StepEntry
    parts.set_matmul_precision()

    class Kit:
        pass
    k = Kit()
    k.parts, k.ops, k.CacheManager, k.BatchBuilder, k.StepEntry = parts, ops, CacheManager, BatchBuilder, StepEntry
    return k


def ctx_for(kit, dtype, page=16, max_tokens=640):
    return kit.parts.BuildContext(dtype, "cuda", max_tokens=max_tokens, max_seqs=8, page_size=page)


def cuts_of(n, sizes):
    """Portions of the given sizes in turn; a last single token joins the portion before it."""
    out, at, i = [], 0, 0
    while at < n:
        c = min(sizes[i % len(sizes)], n - at)
        if n - at - c == 1:
            c += 1
        out.append(c)
        at += c
        i += 1
    return out


class MixerRun:
    def __init__(self, kit, mixer, dtype, page, pages=64, slots=4):
        self.kit, self.mixer, self.dtype = kit, mixer, dtype
        self.need = mixer.cache_need()
        self.cm = kit.CacheManager([self.need], page, pages, slots, dtype=dtype, device="cuda")
        self.bb = kit.BatchBuilder(self.cm, "cuda", query_tiles=getattr(mixer, "query_tiles", lambda: ())())

    def step(self, parts):
        """parts: {sequence: rows [n, width]} -> {sequence: output rows}"""
        for s in parts:
            if s not in self.cm.requests:
                self.cm.admit(s)
        batch = self.bb.build([self.kit.StepEntry(s, [0] * x.shape[0], []) for s, x in parts.items()])
        x = torch.cat(list(parts.values())).cuda().to(self.dtype).contiguous()
        y = self.mixer.forward(x, batch, self.cm.cache_view(0, self.need)).clone()
        out, at = {}, 0
        for s, rows in parts.items():
            out[s] = y[at:at + rows.shape[0]]
            at += rows.shape[0]
        return out

    def feed(self, x, cuts, seq="s", keep=False):
        outs, at = [], 0
        for c in cuts:
            outs.append(self.step({seq: x[at:at + c]})[seq])
            at += c
        assert at == x.shape[0]
        if not keep:
            self.cm.free(seq)
        return torch.cat(outs)

    def plan(self, rows, plan):
        """rows: {sequence: all its rows}; plan: steps {sequence: (lo, hi)} -> {sequence: all outputs}"""
        outs = {s: [] for s in rows}
        for step in plan:
            got = self.step({s: rows[s][lo:hi] for s, (lo, hi) in step.items()})
            for s in step:
                outs[s].append(got[s])
        return {s: torch.cat(v) for s, v in outs.items()}
