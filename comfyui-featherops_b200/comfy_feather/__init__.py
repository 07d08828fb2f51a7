from .loader import FeatherUNetLoader

NODE_CLASS_MAPPINGS = {"FeatherUNetLoader": FeatherUNetLoader}
NODE_DISPLAY_NAME_MAPPINGS = {"FeatherUNetLoader": "Load Diffusion Model (Feather)"}
