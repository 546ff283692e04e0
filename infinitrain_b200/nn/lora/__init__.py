from .lora_config import LoRAConfig, ParseLoRATargetModules
from .lora_layers import LoRAColumnParallelLinear, LoRALinear, LoRARowParallelLinear
from .lora_utils import (CountTotalParameters, CountTrainableParameters, FreezeBaseModel, GetBaseParameters,
                         GetLoRAModel, GetLoRAParameters, InjectLoRALayers, LoadLoRAStateDict, LoadLoRAWeights,
                         LoRAStateDict, MergeAndUnload, MergeLoRAWeights, PrintLoRASummary, ReplaceModuleByPath,
                         SaveLoRAWeights, ShardedLoRAPath, UnfreezeModel, UnmergeLoRAWeights)
