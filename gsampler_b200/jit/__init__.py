"""``gsampler_b200.jit``: trace a sampler written against ``Matrix`` / ``BatchMatrix`` with
torch.fx, rewrite the trace (common subexpressions, relabel + node list merged, slicing + sampling
fused, square + sum fused, paired edge maps merged, a whole GraphSAGE super-batch sampler turned
into one native call), choose sparse formats by measurement, and run the result -- the role of
``gs.jit`` in gSampler (python/gs/jit/{trace,optimize,module}.py), written anew for this
package's operators."""
from . import passes
from .module import compile  # noqa: A001
from .trace import SamplerTracer, trace_sampler

__all__ = ["compile", "passes", "SamplerTracer", "trace_sampler"]
