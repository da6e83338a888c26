"""Key schema of the rendezvous store (reference: ``areal/utils/names.py``)."""
USER = "areal"


def trial_root(experiment_name: str, trial_name: str) -> str:
    return f"{USER}/{experiment_name}/{trial_name}"


def gen_servers(experiment_name: str, trial_name: str) -> str:
    return f"{trial_root(experiment_name, trial_name)}/gen_servers"


def gen_server(experiment_name: str, trial_name: str, server_id: str) -> str:
    return f"{gen_servers(experiment_name, trial_name)}/{server_id}"


def update_weights_from_disk(experiment_name: str, trial_name: str, version: int) -> str:
    return f"{trial_root(experiment_name, trial_name)}/update_weights_from_disk/{version}"


def worker_discovery(experiment_name: str, trial_name: str, role: str, index: int) -> str:
    return f"{trial_root(experiment_name, trial_name)}/workers/{role}/{index}"


def model_version(experiment_name: str, trial_name: str, model_name: str) -> str:
    return f"{trial_root(experiment_name, trial_name)}/model_version/{model_name}"
