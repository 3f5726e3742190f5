class GlobalConfig:
    def __init__(self):
        self.gpu_device_id = 0
        self.bypass_compile_errors = False


global_config = GlobalConfig()
