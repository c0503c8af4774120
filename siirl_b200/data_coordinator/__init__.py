from .data_buffer import DataCoordinator, init_data_coordinator, reset_data_coordinators  # noqa: F401
from .protocol import Batch, all_gather_batch, union_tensor_dict  # noqa: F401
from .sample import (Dict2Samples, Sample, SampleInfo, Samples2Dict, filter_batch, filter_tensordict,  # noqa: F401
                     preprocess_dataloader)
