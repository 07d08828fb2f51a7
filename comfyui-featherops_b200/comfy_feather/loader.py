"""ComfyUI node `FeatherUNetLoader` (reference: comfy_feather/loader.py:9-77): loads a diffusion model with
`custom_operations = feather_ops(out_dtype, excluded_names)` so every eligible Linear becomes a Feather linear.
The reference's loader also installs a sampling-time model pin (comfy_feather/sampling.py:64-83), ComfyUI memory-management
bookkeeping that is not part of the linear path and is not rebuilt here."""

import folder_paths
import torch
from comfy.sd import load_diffusion_model

from .ops import feather_ops

# model_type -> (module-name fragments that stay un-quantised, GEMM output dtype).  Excluded are the non-repeating
# input/output modules and, for qwen, the modulation layers fed by the time-embedding vector.
MODEL_TYPES = {
    "default": ((), torch.bfloat16),
    "anima": (("t_embedder", "x_embedder", "final_layer", "llm_adapter"), torch.bfloat16),
    "flux2": (
        ("img_in", "time_in", "txt_in", "final_layer", "double_stream_modulation_img", "double_stream_modulation_txt", "single_stream_modulation"),
        torch.bfloat16,
    ),
    "qwen": (("time_text_embed", "img_in", "norm_out", "proj_out", "txt_in", "img_mod", "txt_mod"), torch.bfloat16),
    "wan": (("patch_embedding", "text_embedding", "time_embedding", "time_projection", "head"), torch.float16),
}


class FeatherUNetLoader:
    @classmethod
    def INPUT_TYPES(s):
        return {
            "required": {
                "unet_name": (folder_paths.get_filename_list("diffusion_models"),),
                "model_type": (list(MODEL_TYPES),),
            }
        }

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load_unet"
    CATEGORY = "loaders"

    def load_unet(self, unet_name, model_type):
        unet_path = folder_paths.get_full_path_or_raise("diffusion_models", unet_name)
        excluded, out_dtype = MODEL_TYPES.get(model_type, MODEL_TYPES["default"])
        model = load_diffusion_model(unet_path, model_options={"custom_operations": feather_ops(out_dtype=out_dtype, excluded_names=list(excluded))})
        return (model,)
