"""Field names shared by datasets, collators and evaluation (``keys_values/data/constants.py``)."""
INPUT_IDS_NAME = "input_ids"
LABELS_NAME = "labels"
POSITION_NAME = "position"
ORIG_IDX_NAME = "orig_idx"
TASK_NAME = "task"
PAD_DATACASE = {"__pad__": True}


def is_pad_datacase(example) -> bool:
    """Entries appended so that a dataset is a multiple of the batch size."""
    return isinstance(example, dict) and example.get("__pad__", False) is True
