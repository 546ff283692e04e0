from .lora_config import LoRAConfig, ParseLoRATargetModules
from .lora_layers import LoRAColumnParallelLinear, LoRALinear, LoRARowParallelLinear
from .lora_utils import (CountTotalParameters, CountTrainableParameters, FreezeBaseModel, GetBaseParameters,
                         GatherFullLoRAStateDict, GetLoRAModel, GetLoRAParameters, InjectLoRALayers, LoadFullLoRAWeights,
                         LoadLoRAStateDict, LoadLoRAWeights,
                         LoRAStateDict, MergeAndUnload, MergeLoRAWeights, PrintLoRASummary, ReplaceModuleByPath,
                         SaveFullLoRAWeights, SaveLoRAWeights, ScatterFullLoRAStateDict, UnfreezeModel, UnmergeLoRAWeights)
