from mini_train_sys_b200.utils.seed import seed_everything

__all__ = ["seed_everything"]
