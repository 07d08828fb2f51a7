class WrappersMP:
    OUTER_SAMPLE = "outer_sample"
