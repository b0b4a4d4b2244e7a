"""Import stand-in so that the reference's planner (which imports matplotlib.pyplot at module
top for an optional Gantt drawing) can be imported on a machine without matplotlib.  Nothing
here draws."""
