/* Empty stand-in: the PULP board-support header of this name is only included, never used, by the host build of the reference. */
