from .lora import (ARTIFACTS, ExpertLoraAdapters, ParallelDroplessMLP, ParallelMLP, add_expert_lora,
                   get_peft_model, lora_parameters, prepare_peft)
