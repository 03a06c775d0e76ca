import logging


def get_dist_logger(name='stub'):
    return logging.getLogger(name)
