current_loaded_models = []


def free_memory(memory_required, device, keep_loaded=None, *args, **kwargs):
    return []
