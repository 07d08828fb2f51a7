def get_filename_list(folder_name):
    return ["model_a.safetensors", "model_b.safetensors"]


def get_full_path_or_raise(folder_name, filename):
    return f"/models/{folder_name}/{filename}"
