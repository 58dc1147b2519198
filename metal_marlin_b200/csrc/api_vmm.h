// C ABI of the symmetric-memory allocator (symm_vmm.cpp): exportable physical allocations mapped by peer processes and
// NVSwitch multicast objects.  Ids are process-local; negative return values are negated driver error codes.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int mmb_vmm_available(void);                                   // 0: driver API missing; 1: allocations; 2: + multicast objects
long long mmb_vmm_granularity(int dev);
long long mmb_vmm_create(int dev, long long bytes);
int mmb_vmm_export_fd(long long id);
long long mmb_vmm_import_fd(int fd, long long bytes, int dev);
long long mmb_vmm_ptr(long long id);
long long mmb_vmm_size(long long id);
int mmb_vmm_free(long long id);
long long mmb_mc_granularity(int n_dev, long long bytes);
long long mmb_mc_create(int n_dev, long long bytes);
int mmb_mc_export_fd(long long id);
long long mmb_mc_import_fd(int fd, int n_dev, long long bytes);
int mmb_mc_add_device(long long mc, int dev);
int mmb_mc_bind(long long mc, long long mem);
long long mmb_mc_map(long long mc, int dev);
int mmb_mc_unbind(long long mc, int dev, long long mem);
void mmb_close_fd(int fd);
#ifdef __cplusplus
}
#endif
