from .llama import LlamaMeta
from .salepel import SalepelMeta
from .zufadra import ZufadraMeta
from .dumalix import DumalixMeta
from .fugavik import FugavikMeta
from .registry import (Architecture, ConfigError, architecture_for, register_architecture,
                       registered_architectures, unregister_architecture)
