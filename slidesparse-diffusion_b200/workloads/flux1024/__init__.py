"""Constructors for the routed projections of the 'flux1024' workload."""
from .. import prepare_for

WORKLOAD = "flux1024"


def prepare(module, qweight, scales, bias=None, mode="2:4", attention_weight=None, execution="default"):
    return prepare_for(WORKLOAD, module, qweight, scales, bias, mode, attention_weight, execution)
