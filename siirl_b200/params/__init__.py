from .parser import (ConfigError, apply_dict, finalize, get_by_path, load_yaml, merge_node_overrides,  # noqa: F401
                     parse_config, parse_overrides, pretty, set_by_path)
from .schema import *  # noqa: F401,F403
from .schema import SiiRLArguments  # noqa: F401
