from .enums import AdvantageEstimator, AlgorithmType, Role, WorkflowType  # noqa: F401
from .graph_updater import update_task_graph_node_configs  # noqa: F401
from .process_group_manager import ProcessGroupManager  # noqa: F401
from .task_scheduler import TaskScheduler, estimate_graph_model_params, log_schedule_assignments  # noqa: F401
