from .autograd import AutogradEngine, autograd_backward_step
from .base import (
    ADEngine,
    ADResult,
    GradMap,
    LBIBackwardResult,
    ScanBackpropModel,
    assign_grad_map,
    collect_named_grads,
    is_scan_backprop_model,
    store_named_grads,
)
from .local_vjp import LocalVJPProvider, TorchAutogradLocalVJPProvider, surrogate_backward
from .pullbacks import (
    ForwardModeInterfacePullbackProvider,
    InterfacePullbackProvider,
    StructuredInterfacePullbackProvider,
    TorchGraphInterfacePullbackProvider,
    TorchRecomputeInterfacePullbackProvider,
    build_interface_pullback_provider,
    materialize_interface_state_jacobian_t_graph,
    materialize_interface_state_jacobian_t_recompute,
)
from .reference_scan import ReferenceScanEngine, lbi_reference_scan_backward_step
from .scan import ScanADEngine, lbi_scan_backward_step
from .suffix_scan import (
    apply_jacobian_t,
    compose_suffix_jacobian_t,
    interface_state_jacobian_t_stats,
    propagate_state_adjoint_affine,
    propagate_state_adjoint_by_autograd_chain,
    propagate_state_adjoint_by_chain,
    propagate_state_adjoint_from_last_region_input,
    propagate_state_adjoint_with_jacobian_scan,
)

__all__ = [name for name in dir() if not name.startswith("_")]
