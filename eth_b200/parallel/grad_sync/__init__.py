"""Canonical gradient synchronisation across heterogeneous pipelines."""
from .topology import CanonicalTopology, build_canonical_topology  # noqa: F401
from .descriptors import LocalGradientBinding, SerializableGradientDescriptor  # noqa: F401
from .planner import plan_canonical_fragments  # noqa: F401
from .buckets import ProcessGroupRegistry, build_gradient_sync_plan  # noqa: F401
from .executor import GradientBucketExecutor  # noqa: F401
from .manager import GradientSyncManager, initialize_gradient_sync  # noqa: F401
