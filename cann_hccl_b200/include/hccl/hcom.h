/*
 * Group-name ("hcom") front end: communicators addressed by a group string instead of a handle, plus the gradient
 * fusion (bucketing) configuration that data-parallel front ends read.  Thin layer over hccl.h: every group is an
 * ordinary HcclComm (the world group, or a sub-communicator made by HcclCreateSubCommConfig).
 *
 * Role of the reference's framework/hcom/hcom_common.{h,cc} (HcomInitByFile :1339, HcomCreateGroup :383,
 * HcomDestroyGroup :527, HcomGetRankSize :868, HcomGetWorldRankFromGroupRank :700, HcomGetGroupRankFromWorldRank :735,
 * HcomSetGradFusionByIndex :1014, HcomSetGradFusionBySize :1067, HcomGetCommHandleByGroup :171, HcomDestroy :948).
 */
#ifndef HCCL_HCOM_H_
#define HCCL_HCOM_H_

#include "hccl/hccl.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_WORLD_GROUP "hccl_world_group"
#define HCOM_GROUP_NAME_MAX_LENGTH 127

/* Creates the world group from a rank-table file; `identify` is this process's rank id as a decimal string. */
HcclResult HcomInitByFile(const char *rankTablePath, const char *identify);
/* Adopts an existing communicator (for instance one made with HcclCommInitRootInfo) as the world group.  The caller keeps
 * ownership: HcomDestroy forgets it without destroying it.  No counterpart in the reference. */
HcclResult HcomInitByComm(HcclComm worldComm);
/* Destroys every group made through this interface and the world group if HcomInitByFile created it. */
HcclResult HcomDestroy(void);

/* Collective over the ranks of the WORLD group listed in rankIds (world ranks, ascending or not: the position in the list
 * is the group rank).  A rank that is not listed records the membership only. */
HcclResult HcomCreateGroup(const char *group, uint32_t rankNum, uint32_t *rankIds);
HcclResult HcomDestroyGroup(const char *group);

/* group == NULL means the world group in every call below. */
HcclResult HcomGetRankSize(const char *group, uint32_t *rankSize);
HcclResult HcomGetRankId(const char *group, uint32_t *rankId);
HcclResult HcomGetWorldRankFromGroupRank(const char *group, uint32_t groupRank, uint32_t *worldRank);
HcclResult HcomGetGroupRankFromWorldRank(uint32_t worldRank, const char *group, uint32_t *groupRank);
HcclResult HcomGetCommHandleByGroup(const char *group, HcclComm *commHandle);
HcclResult HcomGetTopoDesc(const char *group, HcclTopoDescs *topoDescs, uint32_t topoSize);

/* Gradient fusion: how a data-parallel front end cuts the gradient list of a group into fused AllReduce segments.
 * ByIndex: ascending indices of the last gradient of each segment.  BySize: percentages that sum to 100. */
HcclResult HcomSetGradFusionByIndex(const char *group, uint32_t segmentNum, const uint32_t *inputIdxList);
HcclResult HcomSetGradFusionBySize(const char *group, uint32_t segmentNum, const float *sizeList);
/* Read back (no counterpart in the reference, where the graph engine reads the maps directly): *segmentNum holds the
 * capacity of the list on entry and the number of segments on return; HCCL_E_NOT_FOUND when nothing was set. */
HcclResult HcomGetGradFusionByIndex(const char *group, uint32_t *segmentNum, uint32_t *inputIdxList);
HcclResult HcomGetGradFusionBySize(const char *group, uint32_t *segmentNum, float *sizeList);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_HCOM_H_ */
