from enum import Enum


class Modality(Enum):
    IMAGE = "image"
    MULTI_IMAGES = "multi_images"
    VIDEO = "video"
    AUDIO = "audio"

    @classmethod
    def parse(cls, s: str) -> "Modality":
        return cls[s.upper()] if s.upper() in cls.__members__ else cls(s)
