"""Autodiff facade over ``torch.autograd`` with the reference's names (crates/axonml-autograd):
``Variable``, ``backward``, ``no_grad`` / ``enable_grad`` / ``inference_mode``, ``amp.autocast``,
``checkpoint`` / ``checkpoint_sequential`` (real recomputation; the reference's version only runs
under no_grad, checkpoint.rs:70-95), ``numerical_gradient`` / ``gradcheck``."""
from .amp import (AutocastGuard, AutocastPolicy, autocast, autocast_depth, autocast_dtype, disable_autocast,
                  is_autocast_enabled)
from . import functions
from .checkpoint import checkpoint, checkpoint_sequential, estimate_memory_savings, suggest_segments
from .functions import *  # noqa: F401,F403  (the named backward functions)
from .grad_mode import (EnableGradGuard, InferenceModeGuard, NoGradGuard, enable_grad, inference_mode, is_grad_enabled, is_inference_mode, no_grad,
                        set_grad_enabled_context)
from .graph import ComputationGraph, GradFn, GradientFunction, GraphNode, with_graph

GradFnId = int          # identifier of a backward node (grad_fn.rs ``GradFnId``)
from .variable import Variable, backward, gradcheck, numerical_gradient
