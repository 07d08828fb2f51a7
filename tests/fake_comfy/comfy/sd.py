_last_call = {}


def load_diffusion_model(unet_path, model_options=None):
    """Records the call and returns a tiny object with the attributes the loader node touches."""
    _last_call["unet_path"] = unet_path
    _last_call["model_options"] = dict(model_options or {})

    class _Patcher:
        def __init__(self):
            self.wrappers = []

        def add_wrapper_with_key(self, wrapper_type, key, fn):
            self.wrappers.append((wrapper_type, key, fn))

        def remove_wrappers_with_key(self, wrapper_type, key):
            self.wrappers = [w for w in self.wrappers if not (w[0] == wrapper_type and w[1] == key)]

    return _Patcher()
