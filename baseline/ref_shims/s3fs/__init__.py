class S3FileSystem:
    def __init__(self, *a, **k):
        raise RuntimeError("s3fs is not available")
